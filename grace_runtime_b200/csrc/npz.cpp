#include "npz.h"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>

namespace gb {

ModelError bad_array(const std::string &key, const std::string &what)
{
  return ModelError("model array '" + key + "' " + what + "; re-export the model");
}

namespace {

uint16_t rd16(const unsigned char *p) { return (uint16_t) (p[0] | (p[1] << 8)); }
uint32_t rd32(const unsigned char *p) { return (uint32_t) p[0] | ((uint32_t) p[1] << 8) | ((uint32_t) p[2] << 16) | ((uint32_t) p[3] << 24); }
uint64_t rd64(const unsigned char *p) { return (uint64_t) rd32(p) | ((uint64_t) rd32(p + 4) << 32); }

// parses the .npy header dict: {'descr': '<f8', 'fortran_order': False, 'shape': (3, 4), }
void parse_npy(const std::string &member, const unsigned char *p, size_t n, NpyArray &a)
{
  if (n < 10 || std::memcmp(p, "\x93NUMPY", 6) != 0) throw ModelError("member " + member + " is not a .npy array");
  const int major = p[6];
  size_t hlen, hoff;
  if (major == 1) { hlen = rd16(p + 8); hoff = 10; }
  else { if (n < 12) throw ModelError("truncated .npy header in " + member); hlen = rd32(p + 8); hoff = 12; }
  if (hoff + hlen > n) throw ModelError("truncated .npy header in " + member);
  const std::string h((const char *) p + hoff, hlen);
  auto find_val = [&](const char *name) {
    const size_t q = h.find(name);
    if (q == std::string::npos) throw ModelError(std::string(".npy header of ") + member + " lacks " + name);
    return h.find(':', q) + 1;
  };
  {
    size_t q = find_val("'descr'");
    const size_t a0 = h.find('\'', q), a1 = h.find('\'', a0 + 1);
    if (a0 == std::string::npos || a1 == std::string::npos) throw ModelError("bad descr in " + member);
    const std::string d = h.substr(a0 + 1, a1 - a0 - 1);
    if (d.size() < 3) throw ModelError("bad descr in " + member);
    if (d[0] == '>') throw ModelError("member " + member + " is big-endian");
    a.kind = d[1];
    a.word = std::atoi(d.c_str() + 2);
    if (a.kind == 'U') throw ModelError("member " + member + " holds unicode strings; byte strings (|S) expected");
  }
  {
    size_t q = find_val("'fortran_order'");
    while (q < h.size() && h[q] == ' ') q++;
    a.fortran = h.compare(q, 4, "True") == 0;
  }
  {
    size_t q = find_val("'shape'");
    const size_t a0 = h.find('(', q), a1 = h.find(')', a0);
    if (a0 == std::string::npos || a1 == std::string::npos) throw ModelError("bad shape in " + member);
    const std::string s = h.substr(a0 + 1, a1 - a0 - 1);
    a.shape.clear();
    size_t i = 0;
    while (i < s.size()) {
      while (i < s.size() && (s[i] == ' ' || s[i] == ',')) i++;
      if (i >= s.size()) break;
      int64_t v = 0;
      bool any = false;
      while (i < s.size() && s[i] >= '0' && s[i] <= '9') { v = v * 10 + (s[i] - '0'); i++; any = true; }
      if (!any) throw ModelError("bad shape in " + member);
      a.shape.push_back(v);
    }
  }
  const size_t body = hoff + hlen;
  const int64_t cnt = a.size();
  if (a.word <= 0 || cnt < 0 || (uint64_t) cnt * (uint64_t) a.word > n - body)
    throw ModelError("member " + member + " is truncated");
  a.data.assign(p + body, p + body + (size_t) cnt * a.word);
}

}    // namespace

Npz::Npz(const std::string &path) : path_(path)
{
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) throw ModelError("cannot read the model file " + path);
  const std::streamoff fsz = f.tellg();
  if (fsz < 22) throw ModelError("cannot read the model file " + path + ": not a .npz archive");
  std::vector<unsigned char> buf((size_t) fsz);
  f.seekg(0);
  f.read((char *) buf.data(), fsz);
  if (!f) throw ModelError("cannot read the model file " + path);
  const size_t n = buf.size();
  // end of central directory (search backwards over a possible comment)
  size_t eocd = std::string::npos;
  for (size_t q = n - 22;; q--) {
    if (rd32(&buf[q]) == 0x06054b50u) { eocd = q; break; }
    if (q == 0 || n - q > 22 + 65535) break;
  }
  if (eocd == std::string::npos) throw ModelError("cannot read the model file " + path + ": no ZIP directory");
  uint64_t nent = rd16(&buf[eocd + 10]), cdoff = rd32(&buf[eocd + 16]);
  if (nent == 0xFFFF || cdoff == 0xFFFFFFFFu) {    // ZIP64 end of central directory
    if (eocd < 20 || rd32(&buf[eocd - 20]) != 0x07064b50u) throw ModelError("bad ZIP64 locator in " + path);
    const uint64_t e64 = rd64(&buf[eocd - 20 + 8]);
    if (e64 + 56 > n || rd32(&buf[e64]) != 0x06064b50u) throw ModelError("bad ZIP64 directory in " + path);
    nent = rd64(&buf[e64 + 32]);
    cdoff = rd64(&buf[e64 + 48]);
  }
  size_t p = (size_t) cdoff;
  for (uint64_t e = 0; e < nent; e++) {
    if (p + 46 > n || rd32(&buf[p]) != 0x02014b50u) throw ModelError("bad ZIP directory entry in " + path);
    const int method = rd16(&buf[p + 10]);
    uint64_t csize = rd32(&buf[p + 20]), usize = rd32(&buf[p + 24]), lho = rd32(&buf[p + 42]);
    const size_t nlen = rd16(&buf[p + 28]), xlen = rd16(&buf[p + 30]), clen = rd16(&buf[p + 32]);
    if (p + 46 + nlen + xlen + clen > n) throw ModelError("truncated ZIP directory in " + path);
    std::string name((const char *) &buf[p + 46], nlen);
    // ZIP64 extra field: the 0xFFFFFFFF placeholders in order usize, csize, offset
    size_t x = p + 46 + nlen;
    const size_t xend = x + xlen;
    while (x + 4 <= xend) {
      const int id = rd16(&buf[x]), sz = rd16(&buf[x + 2]);
      if (id == 1) {
        size_t y = x + 4;
        if (usize == 0xFFFFFFFFu && y + 8 <= xend) { usize = rd64(&buf[y]); y += 8; }
        if (csize == 0xFFFFFFFFu && y + 8 <= xend) { csize = rd64(&buf[y]); y += 8; }
        if (lho == 0xFFFFFFFFu && y + 8 <= xend) { lho = rd64(&buf[y]); y += 8; }
      }
      x += 4 + sz;
    }
    p += 46 + nlen + xlen + clen;
    if (method != 0) throw ModelError("the model file " + path + " is compressed (member " + name + "); save it with numpy.savez");
    if (lho + 30 > n || rd32(&buf[lho]) != 0x04034b50u) throw ModelError("bad ZIP member header in " + path);
    const size_t lnlen = rd16(&buf[lho + 26]), lxlen = rd16(&buf[lho + 28]);
    const uint64_t dstart = lho + 30 + lnlen + lxlen;
    if (dstart + csize > n || csize != usize) throw ModelError("truncated member " + name + " in " + path);
    std::string key = name;
    if (key.size() > 4 && key.compare(key.size() - 4, 4, ".npy") == 0) key.resize(key.size() - 4);
    NpyArray a;
    parse_npy(name, &buf[dstart], (size_t) csize, a);
    arrays_[key] = std::move(a);
  }
}

const NpyArray *Npz::find(const std::string &key) const
{
  auto it = arrays_.find(key);
  if (it == arrays_.end()) return nullptr;
  const NpyArray &a = it->second;
  if (a.fortran) {
    int dims = 0;
    for (auto d : a.shape) dims += d > 1;
    if (dims > 1) throw ModelError("model array '" + key + "' is stored in Fortran order; re-export it in C order");
  }
  return &a;
}

std::vector<std::string> Npz::keys() const
{
  std::vector<std::string> k;
  for (auto &kv : arrays_) k.push_back(kv.first);
  return k;
}

namespace {
bool is_int(const NpyArray &a) { return (a.kind == 'i' || a.kind == 'u') && (a.word == 1 || a.word == 2 || a.word == 4 || a.word == 8); }
bool int_at(const NpyArray &a, size_t q, int64_t &v)
{
  const unsigned char *p = a.data.data() + q * a.word;
  const bool u = a.kind == 'u';
  switch (a.word) {
    case 1: v = u ? (int64_t) *p : (int64_t) (int8_t) *p; return true;
    case 2: { uint16_t x; std::memcpy(&x, p, 2); v = u ? (int64_t) x : (int64_t) (int16_t) x; return true; }
    case 4: { uint32_t x; std::memcpy(&x, p, 4); v = u ? (int64_t) x : (int64_t) (int32_t) x; return true; }
    default: { uint64_t x; std::memcpy(&x, p, 8); v = (int64_t) x; return !u || x <= (uint64_t) INT64_MAX; }
  }
}
}    // namespace

std::vector<double> Npz::reals(const std::string &key, bool required) const
{
  const NpyArray *a = find(key);
  if (!a) {
    if (required) throw bad_array(key, "is missing from the .npz file");
    return {};
  }
  std::vector<double> v((size_t) a->size());
  if (a->kind == 'f' && a->word == 4) {
    for (size_t q = 0; q < v.size(); q++) { float x; std::memcpy(&x, a->data.data() + 4 * q, 4); v[q] = x; }
  } else if (a->kind == 'f' && a->word == 8) {
    std::memcpy(v.data(), a->data.data(), 8 * v.size());
  } else if (is_int(*a)) {
    for (size_t q = 0; q < v.size(); q++) {
      int64_t x;
      if (!int_at(*a, q, x)) throw bad_array(key, "has an unsupported dtype, expected a float32 or float64 array");
      v[q] = (double) x;
    }
  } else {
    throw bad_array(key, "has an unsupported dtype, expected a float32 or float64 array");
  }
  for (size_t q = 0; q < v.size(); q++)
    if (!std::isfinite(v[q])) throw bad_array(key, "has a non-finite value (NaN / Inf) at " + std::to_string(q));
  return v;
}

std::vector<int> Npz::ints(const std::string &key, bool required) const
{
  const NpyArray *a = find(key);
  if (!a) {
    if (required) throw bad_array(key, "is missing from the .npz file");
    return {};
  }
  std::vector<int> v((size_t) a->size());
  if (a->kind == 'b' && a->word == 1) {
    for (size_t q = 0; q < v.size(); q++) v[q] = a->data[q] != 0;
    return v;
  }
  if (!is_int(*a)) throw bad_array(key, "has a non-integer dtype, expected an integer array");
  for (size_t q = 0; q < v.size(); q++) {
    int64_t x;
    if (!int_at(*a, q, x) || x < INT32_MIN || x > INT32_MAX) throw bad_array(key, "has a value outside the range of int");
    v[q] = (int) x;
  }
  return v;
}

double Npz::real_scalar(const std::string &key, double def) const
{
  const auto v = reals(key, false);
  if (v.empty()) return def;
  return v[0];
}

int Npz::int_scalar(const std::string &key, int def) const
{
  const NpyArray *a = find(key);
  if (!a) return def;
  if (a->kind == 'f') {    // an export that wrote a count as a float: accepted when integral
    const auto v = reals(key);
    if (v.empty() || v[0] != std::floor(v[0])) throw bad_array(key, "is not an integer");
    return (int) v[0];
  }
  const auto v = ints(key);
  if (v.empty()) throw bad_array(key, "is empty");
  return v[0];
}

int Npz::int_in(const std::string &key, int def, int lo, int hi) const
{
  if (!has(key) && (def < lo || def > hi)) throw bad_array(key, "is missing from the .npz file");
  const int v = int_scalar(key, def);
  if (v < lo || v > hi)
    throw bad_array(key, "is " + std::to_string(v) + ", outside [" + std::to_string(lo) + ", " + std::to_string(hi) + "]");
  return v;
}

std::vector<std::string> Npz::names(const std::string &key) const
{
  const NpyArray *a = find(key);
  if (!a) return {};
  if (a->kind != 'S') throw bad_array(key, "is not a byte-string array (|S)");
  std::vector<std::string> out;
  for (int64_t q = 0; q < a->size(); q++) {
    const char *p = (const char *) a->data.data() + q * a->word;
    size_t len = 0;
    while (len < (size_t) a->word && p[len]) len++;
    out.emplace_back(p, len);
  }
  return out;
}

std::vector<int64_t> Npz::shape(const std::string &key) const
{
  const NpyArray *a = find(key);
  if (!a) throw bad_array(key, "is missing from the .npz file");
  return a->shape;
}

void Npz::require_shape(const std::string &key, const std::vector<int64_t> &want) const
{
  const NpyArray *a = find(key);
  if (!a) return;
  if (a->shape != want) {
    auto str = [](const std::vector<int64_t> &s) {
      std::string r = "(";
      for (size_t i = 0; i < s.size(); i++) r += (i ? ", " : "") + std::to_string(s[i]);
      return r + ")";
    };
    throw bad_array(key, "has shape " + str(a->shape) + ", expected " + str(want));
  }
}

}    // namespace gb
