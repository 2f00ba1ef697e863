// Safetensors directory reader: own header parser (the format's header is a flat JSON object), validation of offsets,
// and parallel pread of tensor bytes into caller memory (pinned staging on the Python side).
// Reference: kernels/src/runtime/safetensors.cpp (JSON header parser :40-150, pread_all :19).
#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "blaze/runtime.h"

namespace {

struct Tensor {
  std::string name, dtype;
  std::vector<int64_t> shape;
  int64_t begin = 0, end = 0;
  int file = 0;
};
struct File {
  std::string path;
  int fd = -1;
  int64_t data_off = 0, size = 0;
};
struct Dir {
  std::vector<File> files;
  std::vector<Tensor> tensors;
};

struct Parser {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  std::string str() {
    ws();
    std::string s;
    if (p >= e || *p != '"') { ok = false; return s; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) { ++p; s.push_back(*p == 'n' ? '\n' : *p == 't' ? '\t' : *p); }
      else s.push_back(*p);
      ++p;
    }
    if (p >= e) ok = false; else ++p;
    return s;
  }
  int64_t num() {
    ws();
    int64_t v = 0;
    bool any = false;
    while (p < e && *p >= '0' && *p <= '9') { v = v * 10 + (*p - '0'); ++p; any = true; }
    if (!any) ok = false;
    return v;
  }
  void skip() {   // skip any JSON value
    ws();
    if (p >= e) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      int depth = 0;
      bool in_s = false;
      while (p < e) {
        if (in_s) { if (*p == '\\') ++p; else if (*p == '"') in_s = false; }
        else if (*p == '"') in_s = true;
        else if (*p == open) ++depth;
        else if (*p == close && --depth == 0) { ++p; return; }
        ++p;
      }
      ok = false;
      return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};

int dtype_size(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2" || d == "F8_E8M0") return 1;
  return 0;
}

bool parse_file(Dir& d, int fi, std::string& err) {
  File& f = d.files[fi];
  uint64_t hlen = 0;
  if (pread(f.fd, &hlen, 8, 0) != 8 || hlen > (uint64_t)f.size - 8 || hlen > (100u << 20)) { err = f.path + ": bad header length"; return false; }
  std::string hdr(hlen, '\0');
  if (pread(f.fd, hdr.data(), hlen, 8) != (ssize_t)hlen) { err = f.path + ": short header"; return false; }
  f.data_off = 8 + (int64_t)hlen;
  Parser ps{hdr.data(), hdr.data() + hdr.size()};
  if (!ps.eat('{')) { err = f.path + ": header is not an object"; return false; }
  while (ps.ok) {
    ps.ws();
    if (ps.eat('}')) break;
    std::string key = ps.str();
    if (!ps.eat(':')) { ps.ok = false; break; }
    if (key == "__metadata__") { ps.skip(); ps.eat(','); continue; }
    Tensor t;
    t.name = key;
    t.file = fi;
    if (!ps.eat('{')) { ps.ok = false; break; }
    while (ps.ok) {
      if (ps.eat('}')) break;
      std::string k = ps.str();
      if (!ps.eat(':')) { ps.ok = false; break; }
      if (k == "dtype") t.dtype = ps.str();
      else if (k == "shape") {
        if (!ps.eat('[')) { ps.ok = false; break; }
        while (ps.ok && !ps.eat(']')) { t.shape.push_back(ps.num()); ps.eat(','); }
      } else if (k == "data_offsets") {
        if (!ps.eat('[')) { ps.ok = false; break; }
        t.begin = ps.num(); ps.eat(','); t.end = ps.num();
        if (!ps.eat(']')) ps.ok = false;
      } else ps.skip();
      ps.eat(',');
    }
    ps.eat(',');
    if (t.shape.size() > 8) { err = f.path + ": tensor " + t.name + " has more than 8 dimensions"; return false; }
    const int es = dtype_size(t.dtype);
    int64_t n = es;
    bool sane = es > 0 && t.begin >= 0 && t.begin <= t.end;
    for (int64_t s : t.shape) {
      // every dimension is bounded by the file size, and the running product is checked for overflow
      if (s < 0 || __builtin_mul_overflow(n, s, &n)) { sane = false; break; }
    }
    if (!sane || t.end - t.begin != n || t.end > f.size - f.data_off) { err = f.path + ": tensor " + t.name + " has inconsistent offsets"; return false; }
    d.tensors.push_back(std::move(t));
  }
  if (!ps.ok) { err = f.path + ": malformed header"; return false; }
  return true;
}

int pread_all(int fd, char* dst, int64_t n, int64_t off) {
  while (n > 0) {
    ssize_t r = pread(fd, dst, (size_t)std::min<int64_t>(n, 1 << 30), off);
    if (r < 0) { if (errno == EINTR) continue; return -errno; }
    if (r == 0) return -EIO;
    dst += r; off += r; n -= r;
  }
  return 0;
}

}  // namespace

extern "C" void* blz_st_open(const char* dir, char* err, int err_len) {
  auto fail = [&](const std::string& m) -> void* { if (err && err_len > 0) snprintf(err, err_len, "%s", m.c_str()); return nullptr; };
  DIR* dp = opendir(dir);
  if (!dp) return fail(std::string("cannot open ") + dir);
  std::vector<std::string> names;
  while (dirent* de = readdir(dp)) {
    std::string n = de->d_name;
    if (n.size() > 12 && n.substr(n.size() - 12) == ".safetensors") names.push_back(n);
  }
  closedir(dp);
  std::sort(names.begin(), names.end());
  if (names.empty()) return fail(std::string("no *.safetensors under ") + dir);
  Dir* d = new Dir();
  std::string e;
  for (size_t i = 0; i < names.size(); ++i) {
    File f;
    f.path = std::string(dir) + "/" + names[i];
    f.fd = open(f.path.c_str(), O_RDONLY);
    struct stat st;
    if (f.fd < 0 || fstat(f.fd, &st) != 0 || st.st_size < 8) {
      if (f.fd >= 0) close(f.fd);       // not yet owned by d->files
      blz_st_close(d);
      return fail(f.path + ": cannot open");
    }
    f.size = st.st_size;
    d->files.push_back(f);
    if (!parse_file(*d, (int)i, e)) { blz_st_close(d); return fail(e); }
  }
  std::sort(d->tensors.begin(), d->tensors.end(), [](const Tensor& a, const Tensor& b) { return a.name < b.name; });
  for (size_t i = 1; i < d->tensors.size(); ++i)
    if (d->tensors[i].name == d->tensors[i - 1].name) { e = "tensor " + d->tensors[i].name + " appears in two shards"; blz_st_close(d); return fail(e); }
  return d;
}

extern "C" void blz_st_close(void* h) {
  Dir* d = reinterpret_cast<Dir*>(h);
  if (!d) return;
  for (File& f : d->files) if (f.fd >= 0) close(f.fd);
  delete d;
}

extern "C" int blz_st_count(void* h) { return (int)reinterpret_cast<Dir*>(h)->tensors.size(); }

extern "C" int blz_st_info(void* h, int i, char* name, int name_len, char* dtype, int dtype_len, int64_t* shape, int64_t* nbytes) {
  Dir* d = reinterpret_cast<Dir*>(h);
  if (i < 0 || i >= (int)d->tensors.size()) return -1;
  const Tensor& t = d->tensors[i];
  if (name) snprintf(name, name_len, "%s", t.name.c_str());
  if (dtype) snprintf(dtype, dtype_len, "%s", t.dtype.c_str());
  for (size_t k = 0; k < t.shape.size() && k < 8; ++k) shape[k] = t.shape[k];
  if (nbytes) *nbytes = t.end - t.begin;
  return (int)t.shape.size();
}

extern "C" int blz_st_find(void* h, const char* name) {
  Dir* d = reinterpret_cast<Dir*>(h);
  auto it = std::lower_bound(d->tensors.begin(), d->tensors.end(), std::string(name),
                             [](const Tensor& t, const std::string& n) { return t.name < n; });
  return (it != d->tensors.end() && it->name == name) ? (int)(it - d->tensors.begin()) : -1;
}

extern "C" int blz_st_read(void* h, int i, void* dst, int64_t dst_bytes, int threads) {
  Dir* d = reinterpret_cast<Dir*>(h);
  if (i < 0 || i >= (int)d->tensors.size()) return -EINVAL;
  const Tensor& t = d->tensors[i];
  const int64_t n = t.end - t.begin;
  if (n != dst_bytes) return -EINVAL;
  const File& f = d->files[t.file];
  const int64_t base = f.data_off + t.begin;
  threads = std::max(1, std::min(threads, (int)(n / (8 << 20)) + 1));
  if (threads == 1) return pread_all(f.fd, (char*)dst, n, base);
  std::vector<std::thread> th;
  std::vector<int> rc(threads, 0);
  const int64_t per = (n + threads - 1) / threads;
  for (int k = 0; k < threads; ++k) {
    const int64_t lo = k * per, hi = std::min(n, lo + per);
    if (lo >= hi) break;
    th.emplace_back([&, k, lo, hi] { rc[k] = pread_all(f.fd, (char*)dst + lo, hi - lo, base + lo); });
  }
  for (auto& x : th) x.join();
  for (int r : rc) if (r) return r;
  return 0;
}
