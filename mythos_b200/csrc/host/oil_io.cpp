// .oil container, SHA-256 and the sidecar check. Layout and semantics are documented in
// mythos_b200/oil/container.py; this is the native implementation used for large files.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "oil_host.h"

namespace {
thread_local std::string g_err;
int fail(int code, const std::string& m) { g_err = m; return code; }

// ------------------------------------------------------------------ SHA-256 (FIPS 180-4)
struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                     0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(h, init, sizeof(h));
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t K[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98,
        0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786,
        0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8,
        0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13,
        0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819,
        0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a,
        0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
        0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | p[4 * i + 1] << 16 | p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
      const uint32_t t1 = hh + S1 + ch + K[i] + w[i];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + S0 + mj;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const uint8_t* p, size_t n) {
    len += n;
    while (n > 0) {
      const size_t take = std::min(n, (size_t)64 - fill);
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  void finish(uint8_t out[32]) {
    const uint64_t bits = len * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    uint8_t lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(lenb, 8);
    for (int i = 0; i < 8; ++i) { out[4 * i] = h[i] >> 24; out[4 * i + 1] = h[i] >> 16; out[4 * i + 2] = h[i] >> 8; out[4 * i + 3] = h[i]; }
  }
};

float half_to_float(uint16_t v) {
  const uint32_t s = (v >> 15) & 1, e = (v >> 10) & 0x1F, m = v & 0x3FF;
  uint32_t bits;
  if (e == 0) {
    if (m == 0) bits = s << 31;
    else {
      int sh = 0; uint32_t mm = m;
      while (!(mm & 0x400)) { mm <<= 1; ++sh; }
      bits = (s << 31) | ((uint32_t)(113 - sh) << 23) | ((mm & 0x3FF) << 13);
    }
  } else if (e == 31) bits = (s << 31) | 0x7F800000u | (m << 13);
  else bits = (s << 31) | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &bits, 4); return f;
}

template <typename T> T rd(const uint8_t* p) { T v; memcpy(&v, p, sizeof(T)); return v; }
}  // namespace

struct OilFile {
  int fd = -1;
  const uint8_t* data = nullptr;
  size_t size = 0;
  uint32_t version = 0, flags = 0, config_size = 0;
  std::vector<uint8_t> fmt;
  std::vector<uint64_t> off;      // block offsets (+ end)
  std::vector<uint32_t> nw;
  struct T { std::string name; uint32_t start, count; };
  std::vector<T> tensors;
  std::map<std::string, uint32_t> by_name;
};

extern "C" {

const char* oil_last_error(void) { return g_err.c_str(); }

void oil_sha256(const uint8_t* data, size_t n, uint8_t out[32]) { Sha256 s; s.update(data, n); s.finish(out); }

int oil_sha256_file(const char* path, uint8_t out[32]) {
  FILE* f = fopen(path, "rb");
  if (!f) return fail(-1, std::string("cannot open ") + path);
  Sha256 s;
  std::vector<uint8_t> buf(1 << 20);
  size_t n;
  while ((n = fread(buf.data(), 1, buf.size(), f)) > 0) s.update(buf.data(), n);
  fclose(f);
  s.finish(out);
  return 0;
}

OilFile* oil_open(const char* path) {
  const int fd = open(path, O_RDONLY);
  if (fd < 0) { fail(-1, std::string("cannot open ") + path); return nullptr; }
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 16) { close(fd); fail(-1, "file too small for an OIL1 header"); return nullptr; }
  void* m = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) { close(fd); fail(-1, "mmap failed"); return nullptr; }
  auto* f = new OilFile;
  f->fd = fd; f->data = (const uint8_t*)m; f->size = st.st_size;
  auto bad = [&](const std::string& why) { fail(-2, std::string(path) + ": " + why); oil_close(f); return (OilFile*)nullptr; };
  if (memcmp(f->data, "OIL1", 4) != 0) return bad("not an OIL1 container");
  f->version = rd<uint32_t>(f->data + 4); f->flags = rd<uint32_t>(f->data + 8); f->config_size = rd<uint32_t>(f->data + 12);
  size_t o = 16 + (size_t)f->config_size;
  if (o + 4 > f->size) return bad("truncated in config");
  const uint32_t nb = rd<uint32_t>(f->data + o); o += 4;
  if (o + 9ull * nb > f->size) return bad("truncated in format table");
  f->fmt.resize(nb);
  for (uint32_t i = 0; i < nb; ++i) f->fmt[i] = f->data[o + 9ull * i + 4];
  o += 9ull * nb;
  if (o + 4 > f->size) return bad("truncated in tensor table");
  const uint32_t nt = rd<uint32_t>(f->data + o); o += 4;
  for (uint32_t i = 0; i < nt; ++i) {
    if (o + 2 > f->size) return bad("truncated in tensor table");
    const uint16_t ln = rd<uint16_t>(f->data + o); o += 2;
    if (o + ln + 8 > f->size) return bad("truncated in tensor table");
    OilFile::T t;
    t.name.assign((const char*)f->data + o, ln); o += ln;
    t.start = rd<uint32_t>(f->data + o); t.count = rd<uint32_t>(f->data + o + 4); o += 8;
    if ((uint64_t)t.start + (uint64_t)t.count > (uint64_t)nb)
      return bad("tensor '" + t.name + "' refers to blocks beyond the block table");
    f->by_name[t.name] = (uint32_t)f->tensors.size();
    f->tensors.push_back(t);
  }
  f->off.resize(nb + 1); f->nw.resize(nb);
  for (uint32_t b = 0; b < nb; ++b) {
    f->off[b] = o;
    if (o + 8 > f->size) return bad("truncated in block " + std::to_string(b));
    f->nw[b] = rd<uint32_t>(f->data + o);
    const uint32_t cb = rd<uint32_t>(f->data + o + 4);
    if ((uint64_t)o + 12ull + cb > f->size) return bad("truncated in block " + std::to_string(b));
    const uint32_t ib = rd<uint32_t>(f->data + o + 8 + cb);
    if ((uint64_t)o + 12ull + cb + ib > f->size) return bad("truncated in block " + std::to_string(b));
    o += 12ull + cb + ib;
  }
  f->off[nb] = o;
  return f;
}

void oil_close(OilFile* f) {
  if (!f) return;
  if (f->data) munmap((void*)f->data, f->size);
  if (f->fd >= 0) close(f->fd);
  delete f;
}
uint32_t oil_version(const OilFile* f) { return f->version; }
uint32_t oil_config_size(const OilFile* f) { return f->config_size; }
const uint8_t* oil_config(const OilFile* f) { return f->data + 16; }
uint32_t oil_num_tensors(const OilFile* f) { return (uint32_t)f->tensors.size(); }
uint32_t oil_num_blocks(const OilFile* f) { return (uint32_t)f->fmt.size(); }
const char* oil_tensor_name(const OilFile* f, uint32_t i) { return i < f->tensors.size() ? f->tensors[i].name.c_str() : nullptr; }

int64_t oil_tensor_numel(const OilFile* f, const char* name) {
  auto it = f->by_name.find(name);
  if (it == f->by_name.end()) return fail(-3, std::string("no tensor named ") + name);
  const auto& t = f->tensors[it->second];
  int64_t n = 0;
  for (uint32_t b = t.start; b < t.start + t.count && b < f->nw.size(); ++b) n += f->nw[b];
  return n;
}

int oil_block_info(const OilFile* f, uint32_t b, uint8_t* format, uint32_t* num_weights, uint64_t* offset,
                   uint32_t* cb_bytes, uint32_t* idx_bytes) {
  if (b >= f->fmt.size()) return fail(-3, "block out of range");
  const uint8_t* p = f->data + f->off[b];
  const uint32_t cb = rd<uint32_t>(p + 4);
  if (format) *format = f->fmt[b];
  if (num_weights) *num_weights = f->nw[b];
  if (offset) *offset = f->off[b];
  if (cb_bytes) *cb_bytes = cb;
  if (idx_bytes) *idx_bytes = rd<uint32_t>(p + 8 + cb);
  return 0;
}

int64_t oil_read_tensor_f32(const OilFile* f, const char* name, float* out, int64_t capacity) {
  auto it = f->by_name.find(name);
  if (it == f->by_name.end()) return fail(-3, std::string("no tensor named ") + name);
  const auto& t = f->tensors[it->second];
  int64_t pos = 0;
  for (uint32_t b = t.start; b < t.start + t.count && b < f->fmt.size(); ++b) {
    const uint8_t* p = f->data + f->off[b];
    const uint32_t n = f->nw[b], cbn = rd<uint32_t>(p + 4);
    const uint8_t* cb = p + 8;
    const uint32_t ibn = rd<uint32_t>(p + 8 + cbn);
    const uint8_t* idx = p + 12 + cbn;
    if (pos + n > capacity) return fail(-4, "output buffer too small");
    float* o = out + pos;
    const uint8_t fmt = f->fmt[b];
    // bytes of index data that the block's format needs for n weights; the header's idx_bytes was
    // checked against the file size in oil_open, so idx[0 .. ibn) is inside the mapping
    const uint64_t bits = fmt == 3 ? 8 : fmt == 2 ? 4 : fmt == 1 ? 2 : fmt == 0 ? 1 : fmt == 4 ? 16 : 32;
    if ((uint64_t)ibn < ((uint64_t)n * bits + 7) / 8)
      return fail(-2, "block " + std::to_string(b) + " of '" + t.name + "': index data shorter than its weight count needs");
    if ((fmt == 3 && cbn < 1028) || (fmt == 2 && cbn < 36))
      return fail(-2, "block " + std::to_string(b) + " of '" + t.name + "': codebook too small for its format");
    if (fmt == 3) {                           // OIL8: magic + 256 f32
      for (uint32_t j = 0; j < n; ++j) o[j] = rd<float>(cb + 4 + 4u * idx[j]);
    } else if (fmt == 2) {       // OIL4: magic + 16 f16, even index in the low nibble
      float c[16];
      for (int k = 0; k < 16; ++k) c[k] = half_to_float(rd<uint16_t>(cb + 4 + 2 * k));
      for (uint32_t j = 0; j < n; ++j) o[j] = c[(j & 1) ? (idx[j >> 1] >> 4) : (idx[j >> 1] & 0xF)];
    } else if (fmt == 1) {                    // ternary: cb = {-s, 0, +s}, 2-bit codes LSB first
      float c[3] = {-1.f, 0.f, 1.f};
      if (cbn >= 12) memcpy(c, cb, 12);
      for (uint32_t j = 0; j < n; ++j) { const int code = (idx[j >> 2] >> (2 * (j & 3))) & 3; o[j] = c[code > 2 ? 2 : code]; }
    } else if (fmt == 0) {                    // binary: cb = {-s, +s}, one bit per weight LSB first
      float c[2] = {-1.f, 1.f};
      if (cbn >= 8) memcpy(c, cb, 8);
      for (uint32_t j = 0; j < n; ++j) o[j] = c[(idx[j >> 3] >> (j & 7)) & 1];
    } else if (fmt == 4) {                    // FP16
      for (uint32_t j = 0; j < n; ++j) o[j] = half_to_float(rd<uint16_t>(idx + 2 * j));
    } else {                                  // FP32 (and unknown codes, as the reference)
      memcpy(o, idx, 4ull * n);
    }
    pos += n;
  }
  return pos;
}

int oil_tensor_sha256(const OilFile* f, const char* name, uint8_t out[32]) {
  auto it = f->by_name.find(name);
  if (it == f->by_name.end()) return fail(-3, std::string("no tensor named ") + name);
  const auto& t = f->tensors[it->second];
  if ((uint64_t)t.start + t.count >= f->off.size()) return fail(-2, std::string("tensor '") + name + "' refers to blocks beyond the block table");
  const uint64_t lo = f->off[t.start], hi = f->off[t.start + t.count];
  oil_sha256(f->data + lo, hi - lo, out);
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------ writer
struct OilWriter {
  std::string path;
  std::vector<uint8_t> header;
  struct B { uint8_t fmt; uint32_t nw; std::vector<uint8_t> cb, idx; };
  std::vector<B> blocks;
  struct T { std::string name; uint32_t start, count; };
  std::vector<T> tensors;
};

extern "C" {

OilWriter* oil_writer_create(const char* path, const uint8_t* config, uint32_t config_size, uint32_t version,
                             uint32_t flags) {
  auto* w = new OilWriter;
  w->path = path;
  w->header.assign({'O', 'I', 'L', '1'});
  auto put32 = [&](uint32_t v) { for (int i = 0; i < 4; ++i) w->header.push_back((uint8_t)(v >> (8 * i))); };
  put32(version); put32(flags); put32(config_size);
  if (config_size) w->header.insert(w->header.end(), config, config + config_size);
  return w;
}
int oil_writer_add_tensor(OilWriter* w, const char* name) {
  w->tensors.push_back({name, (uint32_t)w->blocks.size(), 0});
  return 0;
}
int oil_writer_add_block(OilWriter* w, uint8_t format, uint32_t num_weights, const uint8_t* cb, uint32_t cb_bytes,
                         const uint8_t* idx, uint32_t idx_bytes) {
  if (w->tensors.empty()) return fail(-5, "add a tensor before its blocks");
  OilWriter::B b;
  b.fmt = format; b.nw = num_weights;
  if (cb_bytes) b.cb.assign(cb, cb + cb_bytes);
  if (idx_bytes) b.idx.assign(idx, idx + idx_bytes);
  w->blocks.push_back(std::move(b));
  w->tensors.back().count++;
  return 0;
}
int oil_writer_finish(OilWriter* w) {
  const std::string tmp = w->path + ".tmp";
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) { const int rc = fail(-1, "cannot create " + tmp); delete w; return rc; }
  auto w32 = [&](uint32_t v) { fwrite(&v, 4, 1, f); };
  fwrite(w->header.data(), 1, w->header.size(), f);
  w32((uint32_t)w->blocks.size());
  for (uint32_t i = 0; i < w->blocks.size(); ++i) {
    w32(i); fwrite(&w->blocks[i].fmt, 1, 1, f); w32((uint32_t)w->blocks[i].cb.size());
  }
  w32((uint32_t)w->tensors.size());
  for (const auto& t : w->tensors) {
    const uint16_t ln = (uint16_t)t.name.size();
    fwrite(&ln, 2, 1, f); fwrite(t.name.data(), 1, ln, f); w32(t.start); w32(t.count);
  }
  for (const auto& b : w->blocks) {
    w32(b.nw); w32((uint32_t)b.cb.size()); if (!b.cb.empty()) fwrite(b.cb.data(), 1, b.cb.size(), f);
    w32((uint32_t)b.idx.size()); if (!b.idx.empty()) fwrite(b.idx.data(), 1, b.idx.size(), f);
  }
  fflush(f); fsync(fileno(f)); fclose(f);
  const int rc = rename(tmp.c_str(), w->path.c_str()) == 0 ? 0 : fail(-1, "rename failed");
  delete w;
  return rc;
}

int oil_idx_check(const char* path, char* bad_name, size_t cap) {
  FILE* f = fopen(path, "rb");
  if (!f) return fail(-1000000, std::string("cannot open ") + path);
  std::vector<uint8_t> d;
  uint8_t buf[65536]; size_t n;
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) d.insert(d.end(), buf, buf + n);
  fclose(f);
  if (d.size() < 18 || memcmp(d.data(), "MYTHOSIDX", 9) != 0) return fail(-1000000, "invalid idx file");
  const uint32_t cnt = rd<uint32_t>(d.data() + 14);
  size_t o = 18;
  for (uint32_t i = 0; i < cnt; ++i) {
    if (o + 2 > d.size()) return fail(-(int)(i + 1), "truncated before tensor name length at index " + std::to_string(i));
    const uint16_t ln = rd<uint16_t>(d.data() + o); o += 2;
    if (o + ln + 32 > d.size()) return fail(-(int)(i + 1), "truncated tensor name/hash at index " + std::to_string(i));
    uint8_t h[32];
    oil_sha256(d.data() + o, ln, h);
    if (memcmp(h, d.data() + o + ln, 32) != 0) {
      if (bad_name && cap) { const size_t c = std::min((size_t)ln, cap - 1); memcpy(bad_name, d.data() + o, c); bad_name[c] = 0; }
      return fail(-(int)(i + 1), "name hash mismatch at index " + std::to_string(i));
    }
    o += ln + 32;
  }
  return (int)cnt;
}

}  // extern "C"
