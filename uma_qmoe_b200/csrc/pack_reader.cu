// Native reader of the two on-disk containers of quantised experts and asynchronous staging of one layer.
//
// A pack file is one read-only mapping.  umaq_pack_open checks everything the formats promise before it hands
// out a handle -- the same rules, in the same order and with the same messages as the Python readers of this
// package (pack_files.py), which follow the reference's readers (src/uma_qmoe/expert_pack.py:317-556,
// src/uma_qmoe/target_pack.py:493-812):
//   * 96-byte prefix: magic, version 1, header length, payload offset (a multiple of 4096 behind the header),
//     payload length (to the end of the file), SHA-256 of the header bytes and of the payload;
//   * the header is canonical JSON (sorted keys, "," and ":" separators, ASCII only): parsing it and writing it
//     out again must give the same bytes; zero padding up to the payload;
//   * model identity (for a TargetPack also the policy identity) = SHA-256 of its canonical JSON triple;
//   * tensors in file order without overlap, data at a multiple of the tensor alignment, scales at the next
//     multiple of 4, every gap zero, sizes as the encoding dictates, bits per weight and per-tensor SHA-256 right;
//   * Q4 data never holds the reserved code -8 and has a zero tail nibble; scales are finite and positive.
// Host code only (compiled by nvcc with the rest of the library); the CUDA runtime is used for pinned buffers,
// events and cudaMemcpyAsync -- one call per chunk, nothing batched.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <charconv>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

#if defined(__x86_64__)
#include <cpuid.h>
#include <immintrin.h>
#endif

#include "common.cuh"
#include "umaq_b200.h"

namespace umaq {
namespace {

// ---------------------------------------------------------------------------------------------------
// SHA-256 (FIPS 180-4).  The block function uses the SHA extensions of the CPU when it has them.
// ---------------------------------------------------------------------------------------------------
const uint32_t kK[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

void sha256_blocks_scalar(uint32_t state[8], const uint8_t* data, size_t blocks) {
  for (size_t b = 0; b < blocks; ++b, data += 64) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t)data[4 * i] << 24 | (uint32_t)data[4 * i + 1] << 16 | (uint32_t)data[4 * i + 2] << 8 | data[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = state[0], bb = state[1], c = state[2], d = state[3], e = state[4], f = state[5], g = state[6], h = state[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = h + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + kK[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & bb) ^ (a & c) ^ (bb & c));
      h = g; g = f; f = e; e = d + t1; d = c; c = bb; bb = a; a = t1 + t2;
    }
    state[0] += a; state[1] += bb; state[2] += c; state[3] += d; state[4] += e; state[5] += f; state[6] += g; state[7] += h;
  }
}

#if defined(__x86_64__)
__attribute__((target("sha,sse4.1,ssse3"))) void sha256_blocks_shaext(uint32_t state[8], const uint8_t* data, size_t blocks) {
  const __m128i flip = _mm_set_epi64x(0x0c0d0e0f08090a0bULL, 0x0405060700010203ULL);
  __m128i tmp = _mm_loadu_si128(reinterpret_cast<const __m128i*>(state));        // a b c d
  __m128i st1 = _mm_loadu_si128(reinterpret_cast<const __m128i*>(state + 4));    // e f g h
  tmp = _mm_shuffle_epi32(tmp, 0xB1);                                           // c d a b
  st1 = _mm_shuffle_epi32(st1, 0x1B);                                           // h g f e
  __m128i st0 = _mm_alignr_epi8(tmp, st1, 8);                                   // a b e f
  st1 = _mm_blend_epi16(st1, tmp, 0xF0);                                        // c d g h
  for (size_t b = 0; b < blocks; ++b, data += 64) {
    const __m128i save0 = st0, save1 = st1;
    __m128i m[4];
    for (int i = 0; i < 4; ++i)
      m[i] = _mm_shuffle_epi8(_mm_loadu_si128(reinterpret_cast<const __m128i*>(data + 16 * i)), flip);
    for (int r = 0; r < 16; ++r) {                // four rounds per step
      __m128i cur = m[r & 3];
      __m128i wk = _mm_add_epi32(cur, _mm_loadu_si128(reinterpret_cast<const __m128i*>(kK + 4 * r)));
      st1 = _mm_sha256rnds2_epu32(st1, st0, wk);
      wk = _mm_shuffle_epi32(wk, 0x0E);
      st0 = _mm_sha256rnds2_epu32(st0, st1, wk);
      if (r < 12) {                               // message schedule for step r + 4
        __m128i next = _mm_sha256msg1_epu32(m[r & 3], m[(r + 1) & 3]);
        next = _mm_add_epi32(next, _mm_alignr_epi8(m[(r + 3) & 3], m[(r + 2) & 3], 4));
        m[r & 3] = _mm_sha256msg2_epu32(next, m[(r + 3) & 3]);
      }
    }
    st0 = _mm_add_epi32(st0, save0);
    st1 = _mm_add_epi32(st1, save1);
  }
  tmp = _mm_shuffle_epi32(st0, 0x1B);                                           // f e b a
  st1 = _mm_shuffle_epi32(st1, 0xB1);                                           // d c h g
  st0 = _mm_blend_epi16(tmp, st1, 0xF0);                                        // d c b a
  st1 = _mm_alignr_epi8(st1, tmp, 8);                                           // h g f e
  _mm_storeu_si128(reinterpret_cast<__m128i*>(state), st0);
  _mm_storeu_si128(reinterpret_cast<__m128i*>(state + 4), st1);
}

bool cpu_has_sha() {
  static const bool value = [] {
    unsigned a = 0, b = 0, c = 0, d = 0;
    if (!__get_cpuid_count(7, 0, &a, &b, &c, &d)) return false;
    const bool sha = (b >> 29) & 1u;
    if (!__get_cpuid(1, &a, &b, &c, &d)) return false;
    return sha && ((c >> 19) & 1u) && ((c >> 9) & 1u);       // SSE4.1 and SSSE3
  }();
  return value;
}
#else
bool cpu_has_sha() { return false; }
#endif

struct Sha256 {
  uint32_t state[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  uint8_t pending[64];
  size_t fill = 0;
  uint64_t total = 0;
  bool scalar_only = false;

  void blocks(const uint8_t* data, size_t n) {
#if defined(__x86_64__)
    if (!scalar_only && cpu_has_sha()) { sha256_blocks_shaext(state, data, n); return; }
#endif
    sha256_blocks_scalar(state, data, n);
  }
  void update(const void* src, size_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(src);
    total += n;
    if (fill) {
      const size_t take = std::min(n, 64 - fill);
      std::memcpy(pending + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { blocks(pending, 1); fill = 0; }
    }
    if (n >= 64) { blocks(p, n / 64); p += n / 64 * 64; n %= 64; }
    if (n) { std::memcpy(pending, p, n); fill = n; }
  }
  void finish(uint8_t out[32]) {
    const uint64_t bits = total * 8;
    uint8_t pad[72] = {0x80};
    const size_t padlen = (fill < 56 ? 56 : 120) - fill;
    for (int i = 0; i < 8; ++i) pad[padlen + i] = (uint8_t)(bits >> (56 - 8 * i));
    const uint64_t keep = total;
    update(pad, padlen + 8);
    total = keep;
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) out[4 * i + j] = (uint8_t)(state[i] >> (24 - 8 * j));
  }
};

std::string hex(const uint8_t* bytes, size_t n) {
  static const char* digits = "0123456789abcdef";
  std::string s(2 * n, '0');
  for (size_t i = 0; i < n; ++i) { s[2 * i] = digits[bytes[i] >> 4]; s[2 * i + 1] = digits[bytes[i] & 15]; }
  return s;
}

std::string sha256_hex(const void* a, size_t na, const void* b = nullptr, size_t nb = 0) {
  Sha256 h;
  h.update(a, na);
  if (nb) h.update(b, nb);
  uint8_t d[32];
  h.finish(d);
  return hex(d, 32);
}

// ---------------------------------------------------------------------------------------------------
// JSON: a document tree, a strict parser and the canonical writer (what Python's
// json.dumps(x, sort_keys=True, separators=(",", ":"), allow_nan=False) produces).
// ---------------------------------------------------------------------------------------------------
struct Json {
  enum Type { Null, Bool, Int, Float, String, Array, Object } type = Null;
  bool flag = false;
  long long integer = 0;
  double number = 0.0;
  std::string text;
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> members;

  const Json* get(const char* key) const {
    if (type != Object) return nullptr;
    for (const auto& kv : members)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  bool is_int() const { return type == Int; }
  bool is_str() const { return type == String; }
  bool is_number() const { return type == Int || type == Float; }
  double as_double() const { return type == Int ? (double)integer : number; }
};

struct JsonParser {
  const char* p;
  const char* end;
  int depth = 0;
  bool ok = true;

  void skip() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p; }
  bool fail() { ok = false; return false; }
  bool parse(Json& out) {
    skip();
    if (!value(out)) return false;
    skip();
    return p == end ? true : fail();
  }
  bool literal(const char* word) {
    const size_t n = std::strlen(word);
    if ((size_t)(end - p) < n || std::memcmp(p, word, n) != 0) return fail();
    p += n;
    return true;
  }
  static void utf8(std::string& s, unsigned cp) {
    if (cp < 0x80) s += (char)cp;
    else if (cp < 0x800) { s += (char)(0xC0 | cp >> 6); s += (char)(0x80 | (cp & 63)); }
    else if (cp < 0x10000) { s += (char)(0xE0 | cp >> 12); s += (char)(0x80 | ((cp >> 6) & 63)); s += (char)(0x80 | (cp & 63)); }
    else { s += (char)(0xF0 | cp >> 18); s += (char)(0x80 | ((cp >> 12) & 63)); s += (char)(0x80 | ((cp >> 6) & 63)); s += (char)(0x80 | (cp & 63)); }
  }
  bool hex4(unsigned& v) {
    if (end - p < 4) return fail();
    v = 0;
    for (int i = 0; i < 4; ++i, ++p) {
      const char c = *p;
      v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 99);
      if (v > 0xFFFFF) return fail();
      if (!((c >= '0' && c <= '9') || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F'))) return fail();
    }
    return true;
  }
  bool string(std::string& s) {
    if (p >= end || *p != '"') return fail();
    ++p;
    while (p < end && *p != '"') {
      const unsigned char c = (unsigned char)*p;
      if (c < 0x20) return fail();
      if (c != '\\') { s += *p++; continue; }
      if (++p >= end) return fail();
      switch (*p++) {
        case '"': s += '"'; break;
        case '\\': s += '\\'; break;
        case '/': s += '/'; break;
        case 'b': s += '\b'; break;
        case 'f': s += '\f'; break;
        case 'n': s += '\n'; break;
        case 'r': s += '\r'; break;
        case 't': s += '\t'; break;
        case 'u': {
          unsigned cp;
          if (!hex4(cp)) return false;
          if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
            const char* keep = p;
            p += 2;
            unsigned lo;
            if (!hex4(lo)) return false;
            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            else p = keep;
          }
          utf8(s, cp);
          break;
        }
        default: return fail();
      }
    }
    if (p >= end) return fail();
    ++p;
    return true;
  }
  bool number(Json& out) {
    const char* start = p;
    if (p < end && *p == '-') ++p;
    if (p >= end || *p < '0' || *p > '9') return fail();
    if (*p == '0') ++p; else while (p < end && *p >= '0' && *p <= '9') ++p;
    bool real = false;
    if (p < end && *p == '.') {
      real = true;
      ++p;
      if (p >= end || *p < '0' || *p > '9') return fail();
      while (p < end && *p >= '0' && *p <= '9') ++p;
    }
    if (p < end && (*p == 'e' || *p == 'E')) {
      real = true;
      ++p;
      if (p < end && (*p == '+' || *p == '-')) ++p;
      if (p >= end || *p < '0' || *p > '9') return fail();
      while (p < end && *p >= '0' && *p <= '9') ++p;
    }
    if (real) {
      out.type = Json::Float;
      const auto r = std::from_chars(start, p, out.number);
      return r.ec == std::errc() && r.ptr == p && std::isfinite(out.number) ? true : fail();
    }
    out.type = Json::Int;
    const auto r = std::from_chars(start, p, out.integer);
    return r.ec == std::errc() && r.ptr == p ? true : fail();      // integers beyond 64 bits do not occur in a pack
  }
  bool value(Json& out) {
    if (p >= end || ++depth > 64) return fail();
    bool good = true;
    switch (*p) {
      case 'n': good = literal("null"); out.type = Json::Null; break;
      case 't': good = literal("true"); out.type = Json::Bool; out.flag = true; break;
      case 'f': good = literal("false"); out.type = Json::Bool; out.flag = false; break;
      case '"': out.type = Json::String; good = string(out.text); break;
      case '[': {
        out.type = Json::Array;
        ++p; skip();
        if (p < end && *p == ']') { ++p; break; }
        for (;;) {
          out.items.emplace_back();
          skip();
          if (!value(out.items.back())) return false;
          skip();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == ']') { ++p; break; }
          return fail();
        }
        break;
      }
      case '{': {
        out.type = Json::Object;
        ++p; skip();
        if (p < end && *p == '}') { ++p; break; }
        for (;;) {
          skip();
          std::string key;
          if (!string(key)) return false;
          for (const auto& kv : out.members)
            if (kv.first == key) return fail();               // a repeated key has no canonical form
          skip();
          if (p >= end || *p != ':') return fail();
          ++p; skip();
          out.members.emplace_back(std::move(key), Json());
          if (!value(out.members.back().second)) return false;
          skip();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == '}') { ++p; break; }
          return fail();
        }
        break;
      }
      default: good = number(out);
    }
    --depth;
    return good;
  }
};

void write_string(std::string& out, const std::string& s) {
  static const char* digits = "0123456789abcdef";
  out += '"';
  for (size_t i = 0; i < s.size();) {
    const unsigned char c = (unsigned char)s[i];
    if (c < 0x80) {
      ++i;
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        case '\b': out += "\\b"; break;
        case '\f': out += "\\f"; break;
        default:
          if (c < 0x20 || c == 0x7f) {
            if (c == 0x7f) { out += (char)c; break; }
            out += "\\u00"; out += digits[c >> 4]; out += digits[c & 15];
          } else out += (char)c;
      }
      continue;
    }
    // non-ASCII: \uXXXX escapes, surrogate pairs above the basic plane
    unsigned cp = 0;
    int extra = 0;
    if ((c & 0xE0) == 0xC0) { cp = c & 0x1F; extra = 1; }
    else if ((c & 0xF0) == 0xE0) { cp = c & 0x0F; extra = 2; }
    else { cp = c & 0x07; extra = 3; }
    ++i;
    for (int k = 0; k < extra && i < s.size(); ++k, ++i) cp = (cp << 6) | ((unsigned char)s[i] & 0x3F);
    auto u4 = [&](unsigned v) { out += "\\u"; for (int sh = 12; sh >= 0; sh -= 4) out += digits[(v >> sh) & 15]; };
    if (cp >= 0x10000) { cp -= 0x10000; u4(0xD800 + (cp >> 10)); u4(0xDC00 + (cp & 0x3FF)); }
    else u4(cp);
  }
  out += '"';
}

// repr(float) of Python: the shortest digits that round-trip, fixed notation for exponents in [-4, 16).
void write_float(std::string& out, double v) {
  char buf[40];
  const auto r = std::to_chars(buf, buf + sizeof buf, v, std::chars_format::scientific);
  std::string sci(buf, r.ptr);                     // d[.ddd]e[+-]XX
  const bool neg = sci[0] == '-';
  if (neg) sci.erase(0, 1);
  const size_t e = sci.find('e');
  std::string digits = sci.substr(0, e);
  const int exp10 = std::atoi(sci.c_str() + e + 1);
  digits.erase(std::remove(digits.begin(), digits.end(), '.'), digits.end());
  if (neg) out += '-';
  const int n = (int)digits.size();
  if (exp10 >= -4 && exp10 < 16) {
    if (exp10 < 0) { out += "0."; out.append(-exp10 - 1, '0'); out += digits; }
    else if (n <= exp10 + 1) { out += digits; out.append(exp10 + 1 - n, '0'); out += ".0"; }
    else { out.append(digits, 0, exp10 + 1); out += '.'; out.append(digits, exp10 + 1, std::string::npos); }
  } else {
    out += digits[0];
    if (n > 1) { out += '.'; out.append(digits, 1, std::string::npos); }
    out += 'e';
    out += exp10 < 0 ? '-' : '+';
    const int a = std::abs(exp10);
    if (a < 10) out += '0';
    out += std::to_string(a);
  }
}

void write_canonical(std::string& out, const Json& v) {
  switch (v.type) {
    case Json::Null: out += "null"; break;
    case Json::Bool: out += v.flag ? "true" : "false"; break;
    case Json::Int: out += std::to_string(v.integer); break;
    case Json::Float: write_float(out, v.number); break;
    case Json::String: write_string(out, v.text); break;
    case Json::Array:
      out += '[';
      for (size_t i = 0; i < v.items.size(); ++i) { if (i) out += ','; write_canonical(out, v.items[i]); }
      out += ']';
      break;
    case Json::Object: {
      std::vector<const std::pair<std::string, Json>*> order;
      for (const auto& kv : v.members) order.push_back(&kv);
      std::stable_sort(order.begin(), order.end(), [](auto a, auto b) { return a->first < b->first; });
      out += '{';
      for (size_t i = 0; i < order.size(); ++i) {
        if (i) out += ',';
        write_string(out, order[i]->first);
        out += ':';
        write_canonical(out, order[i]->second);
      }
      out += '}';
      break;
    }
  }
}

std::string canonical(const Json& v) { std::string s; write_canonical(s, v); return s; }

Json json_string(const std::string& s) { Json j; j.type = Json::String; j.text = s; return j; }

// ---------------------------------------------------------------------------------------------------
// The pack
// ---------------------------------------------------------------------------------------------------
struct TensorEntry {
  std::string name;
  int encoding = 0;                  // UMAQ_ENC_*
  long long shape[4] = {0, 0, 0, 0};
  int rank = 0;
  long long elements = 0;
  long long data_offset = 0, data_bytes = 0, scale_offset = 0, scale_bytes = 0;   // relative to the payload
  int layer = -1, expert = -1, projection = -1;                                   // 0 gate, 1 up, 2 down; -1 unknown
};

struct Failure { std::string message; };

}  // namespace
}  // namespace umaq

struct umaq_pack {
  int kind = 0;                      // 0 ExpertPack, 1 TargetPack
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t size = 0;
  std::string header_text;
  umaq::Json header;
  size_t payload_offset = 0, payload_length = 0;
  std::vector<umaq::TensorEntry> tensors;
  std::map<std::string, size_t> by_name;
  std::vector<int> layer_encodings;  // TargetPack policy; ExpertPack: empty (every layer Q4)
  // staging
  std::mutex stage_mutex;
  uint8_t* pinned[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  bool in_use[2] = {false, false};
  cudaStream_t copy_stream = nullptr;
  int staging_device = -1;
  std::atomic<int> tickets{0};

  ~umaq_pack() {
    for (int i = 0; i < 2; ++i) {
      if (done[i]) cudaEventDestroy(done[i]);
      if (pinned[i]) cudaFreeHost(pinned[i]);
    }
    if (copy_stream) cudaStreamDestroy(copy_stream);
    if (map) munmap(const_cast<uint8_t*>(map), size);
    if (fd >= 0) close(fd);
  }
};

struct umaq_stage_ticket {
  umaq_pack* pack = nullptr;
  std::thread worker;
  std::mutex m;
  std::condition_variable cv;
  bool enqueued = false;
  int status = 0;
  std::string error;
  cudaEvent_t finished = nullptr;
  double host_seconds = 0.0;
};

namespace umaq {
namespace {

constexpr size_t kPrefixBytes = 96;
constexpr size_t kPayloadAlignment = 4096;
constexpr size_t kChunkBytes = 32u << 20;         // one pinned buffer
constexpr int kCopyThreads = 8;
const char* kQwenId = "Qwen/Qwen1.5-MoE-A2.7B";
const char* kEncodingNames[3] = {"q4_group128", "q8_group128", "bf16_le"};

[[noreturn]] void reject(const std::string& message) { throw Failure{message}; }

uint32_t le32(const uint8_t* p) { return p[0] | p[1] << 8 | p[2] << 16 | (uint32_t)p[3] << 24; }
uint64_t le64(const uint8_t* p) { return (uint64_t)le32(p) | (uint64_t)le32(p + 4) << 32; }

bool all_zero(const uint8_t* p, size_t n) {
  for (size_t i = 0; i < n; ++i)
    if (p[i]) return false;
  return true;
}

bool positive_int(const Json* v) { return v && v->is_int() && v->integer > 0; }

long long round_up(long long value, const Json* multiple, const char* kind) {
  if (!positive_int(multiple)) reject(std::string(kind) + " alignment must be a positive integer");
  return (value + multiple->integer - 1) / multiple->integer * multiple->integer;
}

std::string quoted(const Json* name) { return "'" + (name && name->is_str() ? name->text : std::string("None")) + "'"; }

bool safe_name(const std::string& s) {
  if (s.empty()) return false;
  for (char c : s)
    if (!((c >= 'A' && c <= 'Z') || (c >= 'a' && c <= 'z') || (c >= '0' && c <= '9') || c == '_' || c == '.' || c == '-')) return false;
  return true;
}

// model.layers.<L>.mlp.experts.<E>.<gate_proj|up_proj|down_proj>.weight
bool parse_expert_name(const std::string& s, int& layer, int& expert, int& projection) {
  auto digits = [&](size_t& i, int& out) {
    const size_t start = i;
    long long v = 0;
    while (i < s.size() && s[i] >= '0' && s[i] <= '9' && i - start < 9) v = v * 10 + (s[i++] - '0');
    out = (int)v;
    return i > start;
  };
  auto word = [&](size_t& i, const char* w) {
    const size_t n = std::strlen(w);
    if (s.compare(i, n, w) != 0) return false;
    i += n;
    return true;
  };
  size_t i = 0;
  if (!word(i, "model.layers.") || !digits(i, layer) || !word(i, ".mlp.experts.") || !digits(i, expert) || !word(i, ".")) return false;
  if (word(i, "gate_proj")) projection = 0;
  else if (word(i, "up_proj")) projection = 1;
  else if (word(i, "down_proj")) projection = 2;
  else return false;
  return word(i, ".weight") && i == s.size();
}

const char* kProjectionNames[3] = {"gate_proj", "up_proj", "down_proj"};

int encoding_id(const std::string& name) {
  for (int i = 0; i < 3; ++i)
    if (name == kEncodingNames[i]) return i;
  return -1;
}

struct Expected { const char *model_id, *revision, *manifest, *policy_id; };

void check_document(umaq_pack& pack, const char* kind, const Expected& expected) {
  const Json& header = pack.header;
  if (pack.kind == 0) {
    const Json* q = header.get("quantization");
    const Json* tensors = header.get("tensors");
    if (!q || q->type != Json::Object || !tensors || tensors->type != Json::Array) reject("ExpertPack header is incomplete");
    const Json* group = q->get("group_size");
    if (!positive_int(group)) reject("ExpertPack quantization contract mismatch");
    const std::string contract = "{\"bits\":4,\"group_size\":" + std::to_string(group->integer) +
                                 ",\"nibble_order\":\"low_first_twos_complement\",\"rounding\":\"nearest_even\","
                                 "\"scale_dtype\":\"float32_le\",\"signed_range\":[-7,7],\"zero_point\":null}";
    if (canonical(*q) != contract) reject("ExpertPack quantization contract mismatch");
    return;
  }
  const Json* format = header.get("format");
  if (!format || !format->is_str() || format->text != "mixed_precision_target_pack") reject("TargetPack header schema is unsupported");
  const Json* policy = header.get("policy");
  if (!policy || policy->type != Json::Object) reject("TargetPack layer policy is invalid");
  const Json* policy_id = policy->get("policy_id");
  if (expected.policy_id && !(policy_id && policy_id->is_str() && policy_id->text == expected.policy_id))
    reject("TargetPack policy id mismatch");
  const Json* model_id = header.get("model")->get("model_id");
  const int layers = model_id && model_id->is_str() && model_id->text == kQwenId ? 24 : 16;
  const Json* table = policy->get("layer_encodings");
  bool complete = table && table->type == Json::Object && (int)table->members.size() == layers;
  pack.layer_encodings.assign(layers, -1);
  if (complete) {
    for (int l = 0; l < layers && complete; ++l) complete = table->get(std::to_string(l).c_str()) != nullptr;
  }
  if (!complete) reject("TargetPack policy must assign every layer exactly once");
  for (int l = 0; l < layers; ++l) {
    const Json* v = table->get(std::to_string(l).c_str());
    const int id = v->is_str() ? encoding_id(v->text) : -1;
    if (id < 0) reject("TargetPack policy contains an unsupported encoding");
    pack.layer_encodings[l] = id;
  }
  if (!policy_id || !policy_id->is_str() || policy_id->text.empty()) reject("TargetPack policy id must be non-empty");
  const Json* evidence = policy->get("policy_evidence_sha256");
  bool hex64 = evidence && evidence->is_str() && evidence->text.size() == 64;
  if (hex64)
    for (char c : evidence->text) hex64 = hex64 && ((c >= '0' && c <= '9') || (c >= 'a' && c <= 'f'));
  if (!hex64) reject("TargetPack policy evidence identity must be SHA-256");
  Json triple;
  triple.type = Json::Object;
  triple.members.emplace_back("policy_id", *policy_id);
  triple.members.emplace_back("layer_encodings", *table);
  triple.members.emplace_back("policy_evidence_sha256", *evidence);
  const std::string text = canonical(triple);
  const std::string identity = sha256_hex(text.data(), text.size());
  const Json* recorded = policy->get("policy_identity_sha256");
  if (policy->members.size() != 4 || !recorded || !recorded->is_str() || recorded->text != identity)
    reject("TargetPack policy identity hash mismatch");
}

// -> encoding id, data bytes, scale bytes of an entry; raises for entry-specific violations
void entry_rules(const umaq_pack& pack, const Json& entry, long long elements, TensorEntry& out) {
  const Json* name = entry.get("name");
  if (pack.kind == 0) {
    const long long group = pack.header.get("quantization")->get("group_size")->integer;
    const long long groups = (elements + group - 1) / group;
    const Json* count = entry.get("group_count");
    if (!count || !count->is_int() || count->integer != groups) reject("ExpertPack tensor " + quoted(name) + " layout is invalid");
    out.encoding = UMAQ_ENC_Q4;
    out.data_bytes = (elements + 1) / 2;
    out.scale_bytes = groups * 4;
    parse_expert_name(name->text, out.layer, out.expert, out.projection);
    return;
  }
  int layer = 0, expert = 0, projection = 0;
  if (!parse_expert_name(name->text, layer, expert, projection)) reject("TargetPack tensor names must be unique fixed OLMoE experts");
  const int layers = (int)pack.layer_encodings.size(), experts = layers == 24 ? 60 : 64;
  const Json *li = entry.get("layer_index"), *ei = entry.get("expert_index"), *pj = entry.get("projection"), *enc = entry.get("encoding");
  const int id = enc && enc->is_str() ? encoding_id(enc->text) : -1;
  if (layer >= layers || expert >= experts || !li || !li->is_int() || li->integer != layer || !ei || !ei->is_int() ||
      ei->integer != expert || !pj || !pj->is_str() || pj->text != kProjectionNames[projection] || id < 0 ||
      id != pack.layer_encodings[layer])
    reject("TargetPack tensor " + quoted(name) + " policy identity is invalid");
  const bool grouped = id != UMAQ_ENC_BF16;
  const long long groups = grouped ? (elements + 127) / 128 : 0;
  const Json *gs = entry.get("group_size"), *gc = entry.get("group_count");
  const bool size_ok = grouped ? (gs && gs->is_int() && gs->integer == 128) : (gs && gs->type == Json::Null);
  if (!size_ok || !gc || !gc->is_int() || gc->integer != groups) reject("TargetPack tensor " + quoted(name) + " layout is invalid");
  out.encoding = id;
  out.data_bytes = id == UMAQ_ENC_Q4 ? (elements + 1) / 2 : id == UMAQ_ENC_Q8 ? elements : elements * 2;
  out.scale_bytes = groups * 4;
  out.layer = layer; out.expert = expert; out.projection = projection;
}

void check_tensors(umaq_pack& pack, const char* kind_c) {
  const std::string kind = kind_c;
  const Json& header = pack.header;
  const Json* entries = header.get("tensors");
  const Json* alignment = header.get("tensor_alignment_bytes");
  round_up(0, alignment, kind_c);
  const Json* count = header.get("tensor_count");
  if (!entries || entries->type != Json::Array || entries->items.empty() || !count || !count->is_int() ||
      count->integer != (long long)entries->items.size())
    reject(kind + " tensor count is inconsistent");
  const char* data_key = pack.kind == 0 ? "packed_offset" : "data_offset";
  const char* size_key = pack.kind == 0 ? "packed_bytes" : "data_bytes";
  const uint8_t* base = pack.map + pack.payload_offset;
  const long long payload_length = (long long)pack.payload_length;
  long long end_of_previous = 0;
  for (const Json& entry : entries->items) {
    if (entry.type != Json::Object) reject(kind + " tensor header must be an object");
    const Json* name = entry.get("name");
    if (!name || !name->is_str() || !safe_name(name->text) || pack.by_name.count(name->text))
      reject(kind + " tensor names must be unique and safe");
    const Json* shape = entry.get("shape");
    bool shape_ok = shape && shape->type == Json::Array && !shape->items.empty() && shape->items.size() <= 4;
    long long elements = 1;
    TensorEntry t;
    t.name = name->text;
    if (shape_ok)
      for (const Json& d : shape->items) {
        shape_ok = shape_ok && d.is_int() && d.integer > 0 && elements <= (1ll << 40);
        if (shape_ok) { t.shape[t.rank++] = d.integer; elements *= d.integer; }
      }
    if (!shape_ok) reject(kind + " tensor " + quoted(name) + " has invalid shape");
    t.elements = elements;
    pack.by_name.emplace(t.name, pack.tensors.size());       // reserved before the rules so that duplicates are seen
    entry_rules(pack, entry, elements, t);
    const Json *start = entry.get(data_key), *scale_at = entry.get("scale_offset"), *end = entry.get("storage_end_offset");
    const Json *ec = entry.get("element_count"), *db = entry.get(size_key), *sb = entry.get("scale_bytes");
    const long long align = alignment->integer;
    bool ok = ec && ec->is_int() && ec->integer == elements && db && db->is_int() && db->integer == t.data_bytes && sb &&
              sb->is_int() && sb->integer == t.scale_bytes && start && start->is_int() && start->integer >= 0 &&
              start->integer % align == 0 && start->integer >= end_of_previous && scale_at && scale_at->is_int() && end &&
              end->is_int();
    if (ok) {
      const long long want_scale = (start->integer + t.data_bytes + 3) / 4 * 4;
      const long long want_end = (want_scale + t.scale_bytes + align - 1) / align * align;
      ok = scale_at->integer == want_scale && end->integer == want_end && want_end <= payload_length;
    }
    if (!ok) reject(kind + " tensor " + quoted(name) + " layout is invalid");
    const Json* bpw = entry.get("effective_bits_per_weight");
    if (!bpw || !bpw->is_number() || bpw->as_double() != (double)((end->integer - start->integer) * 8) / (double)elements)
      reject(kind + " tensor " + quoted(name) + " effective bpw is invalid");
    t.data_offset = start->integer;
    t.scale_offset = scale_at->integer;
    if (!all_zero(base + end_of_previous, start->integer - end_of_previous))
      reject(kind + " tensor " + quoted(name) + " leading gap must be zero");
    if (!all_zero(base + start->integer + t.data_bytes, t.scale_offset - start->integer - t.data_bytes))
      reject(kind + " tensor " + quoted(name) + " data-to-scale gap must be zero");
    if (!all_zero(base + t.scale_offset + t.scale_bytes, end->integer - t.scale_offset - t.scale_bytes))
      reject(kind + " tensor " + quoted(name) + " trailing gap must be zero");
    const uint8_t* data = base + t.data_offset;
    const uint8_t* scales = base + t.scale_offset;
    const Json* digest = entry.get("tensor_payload_sha256");
    if (!digest || !digest->is_str() || digest->text != sha256_hex(data, t.data_bytes, scales, t.scale_bytes))
      reject(kind + " tensor " + quoted(name) + " hash mismatch");
    if (t.encoding == UMAQ_ENC_Q4) {
      // a nibble equal to 8 in either half: (x ^ 0x88) has a zero nibble there
      bool reserved = false;
      for (long long i = 0; i < t.data_bytes && !reserved; ++i) reserved = (data[i] & 0x0F) == 8 || (data[i] >> 4) == 8;
      if (reserved) reject(kind + " tensor " + quoted(name) + " contains reserved Q4 -8");
      if ((elements & 1) && (data[t.data_bytes - 1] >> 4)) reject(kind + " tensor " + quoted(name) + " has non-zero Q4 tail padding");
    }
    for (long long i = 0; i < t.scale_bytes; i += 4) {
      float s;
      std::memcpy(&s, scales + i, 4);
      if (!std::isfinite(s) || !(s > 0.f)) reject(kind + " tensor " + quoted(name) + " scales must be finite and positive");
    }
    end_of_previous = end->integer;
    pack.tensors.push_back(std::move(t));
  }
  if (end_of_previous != payload_length) reject(kind + " payload has unclaimed trailing bytes");
}

void check_totals(const umaq_pack& pack) {
  if (pack.kind == 0) return;
  long long counts[3] = {0, 0, 0};
  for (const TensorEntry& t : pack.tensors) ++counts[t.encoding];
  const Json* recorded = pack.header.get("encoding_tensor_counts");
  bool ok = recorded && recorded->type == Json::Object && recorded->members.size() == 3;
  for (int i = 0; i < 3 && ok; ++i) {
    const Json* v = recorded->get(kEncodingNames[i]);
    ok = v && v->is_int() && v->integer == counts[i];
  }
  if (!ok) reject("TargetPack encoding tensor counts are inconsistent");
}

void open_checked(umaq_pack& pack, const char* path, const Expected& expected) {
  const char* kind = pack.kind == 0 ? "ExpertPack" : "TargetPack";
  const std::string k = kind;
  pack.fd = ::open(path, O_RDONLY | O_CLOEXEC);
  struct stat st {};
  if (pack.fd < 0 || fstat(pack.fd, &st) != 0) reject("cannot map " + k + " " + path + ": " + std::strerror(errno));
  if (st.st_size == 0) reject("cannot map " + k + " " + path + ": cannot mmap an empty file");
  void* view = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_SHARED, pack.fd, 0);
  if (view == MAP_FAILED) reject("cannot map " + k + " " + path + ": " + std::strerror(errno));
  pack.map = static_cast<const uint8_t*>(view);
  pack.size = (size_t)st.st_size;
  if (pack.size < kPrefixBytes) reject(k + " is shorter than its fixed prefix");
  const uint8_t* m = pack.map;
  const char* magic = pack.kind == 0 ? "UQMOEPK1" : "UQMOTPK1";
  const uint32_t version = le32(m + 8), header_len = le32(m + 12);
  const uint64_t offset = le64(m + 16), length = le64(m + 24);
  if (std::memcmp(m, magic, 8) != 0 || version != 1) reject(k + " magic/version mismatch");
  if (offset % kPayloadAlignment || offset < kPrefixBytes + header_len) reject(k + " payload offset/alignment is invalid");
  if (offset + length != pack.size) reject(k + " payload length does not match file size");
  const uint8_t* raw = m + kPrefixBytes;
  uint8_t digest[32];
  { Sha256 h; h.update(raw, header_len); h.finish(digest); }
  if (std::memcmp(digest, m + 32, 32) != 0) reject(k + " header hash mismatch");
  if (!all_zero(m + kPrefixBytes + header_len, offset - kPrefixBytes - header_len)) reject(k + " header padding must be zero");
  { Sha256 h; h.update(m + offset, length); h.finish(digest); }
  if (std::memcmp(digest, m + 64, 32) != 0) reject(k + " payload hash mismatch");
  pack.header_text.assign(reinterpret_cast<const char*>(raw), header_len);
  JsonParser parser{pack.header_text.data(), pack.header_text.data() + pack.header_text.size()};
  if (!parser.parse(pack.header)) reject(k + " header is not canonical JSON");
  if (canonical(pack.header) != pack.header_text) reject(k + " header JSON is not canonical");
  const Json* schema = pack.header.get("schema_version");
  if (pack.header.type != Json::Object || !schema || !schema->is_int() || schema->integer != 1) reject(k + " header schema is unsupported");
  const Json* model = pack.header.get("model");
  if (!model || model->type != Json::Object) reject(k + " header is incomplete");
  Json triple;
  triple.type = Json::Object;
  const char* keys[3] = {"model_id", "model_revision", "model_manifest_sha256"};
  for (const char* key : keys) {
    const Json* v = model->get(key);
    triple.members.emplace_back(key, v ? *v : json_string(""));
  }
  const std::string text = canonical(triple);
  const Json* identity = model->get("model_identity_sha256");
  if (!identity || !identity->is_str() || identity->text != sha256_hex(text.data(), text.size())) reject(k + " model identity hash mismatch");
  const char* wants[3] = {expected.model_id, expected.revision, expected.manifest};
  const char* labels[3] = {"model id", "model revision", "model manifest"};
  for (int i = 0; i < 3; ++i) {
    const Json* v = model->get(keys[i]);
    if (wants[i] && !(v && v->is_str() && v->text == wants[i])) reject(k + " " + labels[i] + " mismatch");
  }
  pack.payload_offset = offset;
  pack.payload_length = length;
  check_document(pack, kind, expected);
  check_tensors(pack, kind);
  check_totals(pack);
}

// ---------------------------------------------------------------------------------------------------
// Staging: mapping -> pinned chunk (several threads) -> cudaMemcpyAsync on the pack's copy stream
// ---------------------------------------------------------------------------------------------------
struct Piece { const uint8_t* src; uint8_t* device_dst; size_t at; size_t bytes; };   // `at`: offset in the pinned buffer

// Fills one pinned buffer from the mapping: the pieces are cut into runs of at most 1 MiB and the runs dealt to
// the copy threads in turn (a layer's tensors are 64 KiB to a few MiB each, so no single piece is worth splitting
// further and no thread is left with all the large ones).
void fill_pinned(uint8_t* pinned, const std::vector<Piece>& pieces) {
  struct Run { const uint8_t* src; uint8_t* dst; size_t bytes; };
  std::vector<Run> runs;
  size_t total = 0;
  for (const Piece& p : pieces)
    for (size_t done = 0; done < p.bytes; done += (1u << 20)) {
      runs.push_back({p.src + done, pinned + p.at + done, std::min(p.bytes - done, (size_t)1 << 20)});
      total += runs.back().bytes;
    }
  const int threads = total < (2u << 20) ? 1 : kCopyThreads;
  auto work = [&runs, threads](int t) {
    for (size_t i = t; i < runs.size(); i += threads) std::memcpy(runs[i].dst, runs[i].src, runs[i].bytes);
  };
  std::vector<std::thread> helpers;
  for (int t = 1; t < threads; ++t) helpers.emplace_back(work, t);
  work(0);
  for (auto& h : helpers) h.join();
}

struct Span { const uint8_t* src; uint8_t* dst; size_t bytes; };

std::string stage_spans(umaq_pack& pack, const std::vector<Span>& spans, int device, cudaEvent_t finished) {
  std::lock_guard<std::mutex> lock(pack.stage_mutex);
  auto cuda = [](cudaError_t e, const char* what) { return e == cudaSuccess ? std::string() : std::string(what) + ": " + cudaGetErrorString(e); };
  std::string err = cuda(cudaSetDevice(device), "cudaSetDevice");
  if (!err.empty()) return err;
  if (pack.staging_device != device) {
    if (pack.staging_device >= 0) return "a pack stages to one device";
    for (int i = 0; i < 2 && err.empty(); ++i) {
      err = cuda(cudaHostAlloc(reinterpret_cast<void**>(&pack.pinned[i]), kChunkBytes, cudaHostAllocDefault), "cudaHostAlloc");
      if (err.empty()) err = cuda(cudaEventCreateWithFlags(&pack.done[i], cudaEventDisableTiming), "cudaEventCreate");
    }
    if (err.empty()) err = cuda(cudaStreamCreateWithFlags(&pack.copy_stream, cudaStreamNonBlocking), "cudaStreamCreate");
    if (!err.empty()) return err;
    pack.staging_device = device;
  }
  // The spans are packed back to back into chunks of the pinned buffers.  A chunk is filled by the copy threads,
  // then sent with one cudaMemcpyAsync per piece (the pieces' destinations differ) and closed with an event; while it
  // travels the other buffer is filled.
  int buffer = 0;
  size_t fill = 0;
  std::vector<Piece> pieces;
  auto flush = [&]() -> std::string {
    fill_pinned(pack.pinned[buffer], pieces);
    for (const Piece& p : pieces) {
      std::string e = cuda(cudaMemcpyAsync(p.device_dst, pack.pinned[buffer] + p.at, p.bytes, cudaMemcpyHostToDevice, pack.copy_stream), "cudaMemcpyAsync");
      if (!e.empty()) return e;
    }
    pieces.clear();
    std::string e = cuda(cudaEventRecord(pack.done[buffer], pack.copy_stream), "cudaEventRecord");
    pack.in_use[buffer] = true;
    buffer ^= 1;
    fill = 0;
    if (e.empty() && pack.in_use[buffer]) e = cuda(cudaEventSynchronize(pack.done[buffer]), "cudaEventSynchronize");
    pack.in_use[buffer] = false;
    return e;
  };
  if (pack.in_use[0]) { err = cuda(cudaEventSynchronize(pack.done[0]), "cudaEventSynchronize"); pack.in_use[0] = false; }
  for (const Span& s : spans) {
    size_t done = 0;
    while (done < s.bytes && err.empty()) {
      const size_t n = std::min(s.bytes - done, kChunkBytes - fill);
      pieces.push_back({s.src + done, s.dst + done, fill, n});
      fill += (n + 255) / 256 * 256;
      done += n;
      if (fill + 256 > kChunkBytes) err = flush();
    }
    if (!err.empty()) return err;
  }
  if (fill && err.empty()) err = flush();
  if (err.empty()) err = cuda(cudaEventRecord(finished, pack.copy_stream), "cudaEventRecord");
  return err;
}

}  // namespace
}  // namespace umaq

// ---------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------
using namespace umaq;

extern "C" int umaq_pack_open(const char* path, int kind, const char* expected_model_id, const char* expected_model_revision,
                              const char* expected_model_manifest_sha256, const char* expected_policy_id, umaq_pack** out) {
  if (!path || !out || kind < 0 || kind > 1) { set_error("pack: needs a path, a kind (0 ExpertPack, 1 TargetPack) and an output"); return ERR_BAD_ARGUMENT; }
  *out = nullptr;
  auto pack = std::make_unique<umaq_pack>();
  pack->kind = kind;
  try {
    open_checked(*pack, path, Expected{expected_model_id, expected_model_revision, expected_model_manifest_sha256, expected_policy_id});
  } catch (const Failure& f) {
    set_error("%s", f.message.c_str());
    return ERR_BAD_ARGUMENT;
  } catch (const std::exception& e) {
    set_error("pack: %s", e.what());
    return ERR_BAD_ARGUMENT;
  }
  *out = pack.release();
  return ERR_NONE;
}

extern "C" void umaq_pack_close(umaq_pack* pack) { delete pack; }

extern "C" long long umaq_pack_tensor_count(const umaq_pack* pack) { return pack ? (long long)pack->tensors.size() : -1; }

extern "C" const char* umaq_pack_header_json(const umaq_pack* pack, size_t* length) {
  if (!pack) return nullptr;
  if (length) *length = pack->header_text.size();
  return pack->header_text.data();
}

extern "C" int umaq_pack_layer_encoding(const umaq_pack* pack, int layer) {
  if (!pack) return ERR_BAD_ARGUMENT;
  if (pack->kind == 0) return UMAQ_ENC_Q4;
  if (layer < 0 || layer >= (int)pack->layer_encodings.size()) {
    set_error("TargetPack layer index must be in [0, %d]", (int)pack->layer_encodings.size() - 1);
    return ERR_BAD_ARGUMENT;
  }
  return pack->layer_encodings[layer];
}

static void fill_view(const umaq_pack* pack, const TensorEntry& t, umaq_pack_tensor* view) {
  const uint8_t* base = pack->map + pack->payload_offset;
  view->name = t.name.c_str();
  view->data = base + t.data_offset;
  view->data_bytes = (size_t)t.data_bytes;
  view->scales = base + t.scale_offset;
  view->scale_bytes = (size_t)t.scale_bytes;
  view->encoding = t.encoding;
  view->rank = t.rank;
  for (int i = 0; i < 4; ++i) view->shape[i] = t.shape[i];
  view->layer = t.layer; view->expert = t.expert; view->projection = t.projection;
}

extern "C" int umaq_pack_tensor_view(const umaq_pack* pack, const char* name, umaq_pack_tensor* view) {
  if (!pack || !name || !view) { set_error("pack: tensor_view needs a pack, a name and an output"); return ERR_BAD_ARGUMENT; }
  const auto it = pack->by_name.find(name);
  if (it == pack->by_name.end()) {
    set_error("%s has no tensor '%s'", pack->kind == 0 ? "ExpertPack" : "TargetPack", name);
    return ERR_BAD_ARGUMENT;
  }
  fill_view(pack, pack->tensors[it->second], view);
  return ERR_NONE;
}

extern "C" int umaq_pack_tensor_at(const umaq_pack* pack, long long index, umaq_pack_tensor* view) {
  if (!pack || !view || index < 0 || index >= (long long)pack->tensors.size()) { set_error("pack: tensor index out of range"); return ERR_BAD_ARGUMENT; }
  fill_view(pack, pack->tensors[(size_t)index], view);
  return ERR_NONE;
}

extern "C" int umaq_sha256(const void* data, size_t bytes, int scalar_only, unsigned char digest[32]) {
  if ((!data && bytes) || !digest) return ERR_BAD_ARGUMENT;
  Sha256 h;
  h.scalar_only = scalar_only != 0;
  h.update(data, bytes);
  h.finish(digest);
  return ERR_NONE;
}

extern "C" int umaq_stage_layer_async(umaq_pack* pack, int layer_index, const umaq_layer* dst, int device, umaq_stage_ticket** out) {
  if (!pack || !dst || !out || !dst->gate || !dst->up || !dst->down) { set_error("stage: needs a pack, a destination layer and a ticket output"); return ERR_BAD_ARGUMENT; }
  *out = nullptr;
  const int E = dst->num_experts, H = dst->hidden, I = dst->intermediate;
  const int enc = pack->kind == 0 ? UMAQ_ENC_Q4 : (layer_index >= 0 && layer_index < (int)pack->layer_encodings.size() ? pack->layer_encodings[layer_index] : -1);
  if (enc < 0 || enc != dst->encoding) { set_error("stage: layer %d of the pack is not encoded as the destination says", layer_index); return ERR_BAD_ARGUMENT; }
  const bool quantised = enc != UMAQ_ENC_BF16;
  if (quantised && (!dst->gate_scales || !dst->up_scales || !dst->down_scales)) { set_error("stage: a quantised layer needs scale destinations"); return ERR_BAD_ARGUMENT; }
  // every expert tensor of the layer, in the staged order: per projection all experts concatenated
  std::vector<Span> spans;
  const uint8_t* base = pack->map + pack->payload_offset;
  // the destination tensors are the caller's, written here on its behalf
  auto writable = [](const void* p) { return static_cast<uint8_t*>(const_cast<void*>(p)); };
  uint8_t* code_dst[3] = {writable(dst->gate), writable(dst->up), writable(dst->down)};
  uint8_t* scale_dst[3] = {writable(dst->gate_scales), writable(dst->up_scales), writable(dst->down_scales)};
  for (int p = 0; p < 3; ++p) {
    const long long rows = p == 2 ? H : I, k = p == 2 ? I : H;
    const long long code_bytes = enc == UMAQ_ENC_Q4 ? rows * k / 2 : enc == UMAQ_ENC_Q8 ? rows * k : rows * k * 2;
    const long long scale_bytes = quantised ? rows * k / 128 * 4 : 0;
    for (int e = 0; e < E; ++e) {
      char name[128];
      std::snprintf(name, sizeof name, "model.layers.%d.mlp.experts.%d.%s.weight", layer_index, e, kProjectionNames[p]);
      const auto it = pack->by_name.find(name);
      if (it == pack->by_name.end()) { set_error("stage: the pack has no tensor '%s'", name); return ERR_BAD_ARGUMENT; }
      const TensorEntry& t = pack->tensors[it->second];
      if (t.rank != 2 || t.shape[0] != rows || t.shape[1] != k || t.encoding != enc || t.data_bytes != code_bytes || t.scale_bytes != scale_bytes) {
        set_error("stage: tensor '%s' does not have the layer's shape and encoding", name);
        return ERR_BAD_ARGUMENT;
      }
      spans.push_back({base + t.data_offset, code_dst[p] + (size_t)e * code_bytes, (size_t)code_bytes});
    }
    if (quantised)
      for (int e = 0; e < E; ++e) {
        char name[128];
        std::snprintf(name, sizeof name, "model.layers.%d.mlp.experts.%d.%s.weight", layer_index, e, kProjectionNames[p]);
        const TensorEntry& t = pack->tensors[pack->by_name.find(name)->second];
        spans.push_back({base + t.scale_offset, scale_dst[p] + (size_t)e * scale_bytes, (size_t)scale_bytes});
      }
  }
  auto ticket = std::make_unique<umaq_stage_ticket>();
  ticket->pack = pack;
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ticket->finished, cudaEventDisableTiming);
  if (e != cudaSuccess) { set_error("stage: %s", cudaGetErrorString(e)); return ERR_LAUNCH; }
  umaq_stage_ticket* raw = ticket.get();
  pack->tickets.fetch_add(1);
  raw->worker = std::thread([raw, pack, spans = std::move(spans), device] {
    const auto t0 = std::chrono::steady_clock::now();
    std::string err = stage_spans(*pack, spans, device, raw->finished);
    std::lock_guard<std::mutex> lock(raw->m);
    raw->host_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    raw->status = err.empty() ? ERR_NONE : ERR_LAUNCH;
    raw->error = err;
    raw->enqueued = true;
    raw->cv.notify_all();
  });
  *out = ticket.release();
  return ERR_NONE;
}

extern "C" int umaq_stage_wait(umaq_stage_ticket* ticket, void* stream, double* host_seconds) {
  if (!ticket) { set_error("stage: no ticket"); return ERR_BAD_ARGUMENT; }
  {
    std::unique_lock<std::mutex> lock(ticket->m);
    ticket->cv.wait(lock, [&] { return ticket->enqueued; });
  }
  ticket->worker.join();
  int status = ticket->status;
  if (status != ERR_NONE) set_error("stage: %s", ticket->error.c_str());
  else if (cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), ticket->finished, 0) != cudaSuccess) {
    set_error("stage: cudaStreamWaitEvent failed");
    status = ERR_LAUNCH;
  }
  if (host_seconds) *host_seconds = ticket->host_seconds;
  // the event must outlive the wait that was just enqueued: destroying it is deferred by the runtime until then
  cudaEventDestroy(ticket->finished);
  ticket->pack->tickets.fetch_sub(1);
  delete ticket;
  return status;
}
