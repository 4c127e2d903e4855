// BPE tokenizer, RNG and page allocator of the host runtime (see oil_host.h).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <queue>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "oil_host.h"

// ------------------------------------------------------------------ BPE
struct OilBpe {
  std::vector<std::string> vocab;
  std::map<std::pair<int, int>, int> merges;
};

namespace {
struct PairHash {
  size_t operator()(const std::pair<int, int>& p) const { return ((size_t)p.first << 32) ^ (size_t)(uint32_t)p.second; }
};
}  // namespace

extern "C" {

OilBpe* oil_bpe_train(const uint8_t* text, size_t n, int vocab_size) {
  auto* t = new OilBpe;
  for (int i = 0; i < 256; ++i) t->vocab.push_back(std::string(1, (char)i));
  if (n < 2 || vocab_size <= 256) return t;
  std::vector<int> ids(text, text + n), prev(n), next(n);
  std::vector<char> alive(n, 1);
  for (size_t i = 0; i < n; ++i) { prev[i] = (int)i - 1; next[i] = (i + 1 < n) ? (int)i + 1 : -1; }
  std::unordered_map<std::pair<int, int>, long long, PairHash> counts;
  std::unordered_map<std::pair<int, int>, std::set<int>, PairHash> where;
  for (size_t i = 0; i + 1 < n; ++i) { auto p = std::make_pair(ids[i], ids[i + 1]); counts[p]++; where[p].insert((int)i); }
  typedef std::pair<long long, std::pair<int, int>> HeapItem;
  auto cmp = [](const HeapItem& a, const HeapItem& b) { return a.first != b.first ? a.first < b.first : a.second > b.second; };
  std::priority_queue<HeapItem, std::vector<HeapItem>, decltype(cmp)> heap(cmp);
  for (auto& kv : counts) heap.push({kv.second, kv.first});
  while ((int)t->vocab.size() < vocab_size && !heap.empty()) {
    auto item = heap.top(); heap.pop();
    auto it = counts.find(item.second);
    const long long c = it == counts.end() ? 0 : it->second;
    if (c <= 0 || c != item.first) { if (c > 0) heap.push({c, item.second}); continue; }
    if (c < 2) break;
    const auto pair = item.second;
    const int id = (int)t->vocab.size();
    t->vocab.push_back(t->vocab[pair.first] + t->vocab[pair.second]);
    t->merges[pair] = id;
    std::set<std::pair<int, int>> touched;
    std::set<int> pos; pos.swap(where[pair]);
    for (int i : pos) {
      const int j = alive[i] ? next[i] : -1;
      if (!alive[i] || j < 0 || !alive[j] || ids[i] != pair.first || ids[j] != pair.second) continue;
      const int pi = prev[i], nj = next[j];
      if (pi >= 0) { auto o = std::make_pair(ids[pi], ids[i]); counts[o]--; where[o].erase(pi); touched.insert(o); }
      if (nj >= 0) { auto o = std::make_pair(ids[j], ids[nj]); counts[o]--; where[o].erase(j); touched.insert(o); }
      ids[i] = id; alive[j] = 0; next[i] = nj;
      if (nj >= 0) prev[nj] = i;
      if (pi >= 0) { auto o = std::make_pair(ids[pi], id); counts[o]++; where[o].insert(pi); touched.insert(o); }
      if (nj >= 0) { auto o = std::make_pair(id, ids[nj]); counts[o]++; where[o].insert(i); touched.insert(o); }
    }
    counts.erase(pair);
    for (auto& p : touched) { auto f = counts.find(p); if (f != counts.end() && f->second > 0) heap.push({f->second, p}); }
  }
  return t;
}

OilBpe* oil_bpe_load(const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) return nullptr;
  auto* t = new OilBpe;
  int vs = 0;
  if (fread(&vs, 4, 1, f) != 1) { fclose(f); delete t; return nullptr; }
  for (int i = 0; i < vs; ++i) {
    int ln = 0;
    if (fread(&ln, 4, 1, f) != 1) break;
    std::string s(ln, '\0');
    if (ln && fread(&s[0], 1, ln, f) != (size_t)ln) break;
    t->vocab.push_back(s);
  }
  int ms = 0;
  if (fread(&ms, 4, 1, f) == 1)
    for (int i = 0; i < ms; ++i) { int abc[3]; if (fread(abc, 4, 3, f) != 3) break; t->merges[{abc[0], abc[1]}] = abc[2]; }
  fclose(f);
  return t;
}

int oil_bpe_save(const OilBpe* t, const char* path) {
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  const int vs = (int)t->vocab.size();
  fwrite(&vs, 4, 1, f);
  for (auto& v : t->vocab) { const int ln = (int)v.size(); fwrite(&ln, 4, 1, f); fwrite(v.data(), 1, ln, f); }
  const int ms = (int)t->merges.size();
  fwrite(&ms, 4, 1, f);
  for (auto& m : t->merges) { const int abc[3] = {m.first.first, m.first.second, m.second}; fwrite(abc, 4, 3, f); }
  fclose(f);
  return 0;
}
void oil_bpe_free(OilBpe* t) { delete t; }
int oil_bpe_vocab_size(const OilBpe* t) { return (int)t->vocab.size(); }

int64_t oil_bpe_encode(const OilBpe* t, const uint8_t* text, size_t n, int32_t* out, int64_t capacity) {
  std::vector<int> ids(text, text + n);
  while (ids.size() > 1 && !t->merges.empty()) {
    int best_rank = -1; std::pair<int, int> best;
    for (size_t i = 0; i + 1 < ids.size(); ++i) {
      auto it = t->merges.find({ids[i], ids[i + 1]});
      if (it != t->merges.end() && (best_rank < 0 || it->second < best_rank)) { best_rank = it->second; best = it->first; }
    }
    if (best_rank < 0) break;
    std::vector<int> next; next.reserve(ids.size());
    for (size_t i = 0; i < ids.size();) {
      if (i + 1 < ids.size() && ids[i] == best.first && ids[i + 1] == best.second) { next.push_back(best_rank); i += 2; }
      else next.push_back(ids[i++]);
    }
    ids.swap(next);
  }
  if ((int64_t)ids.size() > capacity) return -(int64_t)ids.size();
  for (size_t i = 0; i < ids.size(); ++i) out[i] = ids[i];
  return (int64_t)ids.size();
}

int64_t oil_bpe_decode(const OilBpe* t, const int32_t* ids, int64_t n, uint8_t* out, int64_t capacity) {
  int64_t pos = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (ids[i] < 0 || ids[i] >= (int)t->vocab.size()) continue;
    const std::string& s = t->vocab[ids[i]];
    if (pos + (int64_t)s.size() > capacity) return -(pos + (int64_t)s.size());
    memcpy(out + pos, s.data(), s.size()); pos += s.size();
  }
  return pos;
}

}  // extern "C"

// ------------------------------------------------------------------ RNG
struct OilRng { uint64_t s[2]; bool has_spare = false; double spare = 0; };

extern "C" {

OilRng* oil_rng_create(uint64_t seed) {
  auto* r = new OilRng;
  auto splitmix = [&seed]() { uint64_t z = (seed += 0x9E3779B97F4A7C15ull); z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
                              z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31); };
  r->s[0] = splitmix(); r->s[1] = splitmix();
  return r;
}
void oil_rng_free(OilRng* r) { delete r; }
uint64_t oil_rng_next(OilRng* r) {
  const uint64_t s0 = r->s[0]; uint64_t s1 = r->s[1];
  const uint64_t result = s0 + s1;
  s1 ^= s0;
  r->s[0] = ((s0 << 24) | (s0 >> 40)) ^ s1 ^ (s1 << 16);
  r->s[1] = (s1 << 37) | (s1 >> 27);
  return result;
}
double oil_rng_uniform(OilRng* r) { return (double)(oil_rng_next(r) >> 11) * (1.0 / 9007199254740992.0); }
double oil_rng_normal(OilRng* r) {
  if (r->has_spare) { r->has_spare = false; return r->spare; }
  double u1 = oil_rng_uniform(r), u2 = oil_rng_uniform(r);
  if (u1 < 1e-300) u1 = 1e-300;
  const double m = std::sqrt(-2.0 * std::log(u1));
  r->spare = m * std::sin(6.283185307179586 * u2); r->has_spare = true;
  return m * std::cos(6.283185307179586 * u2);
}
void oil_rng_fill_uniform(OilRng* r, float* out, int64_t n, float lo, float hi) {
  for (int64_t i = 0; i < n; ++i) out[i] = lo + (hi - lo) * (float)oil_rng_uniform(r);
}

}  // extern "C"

// ------------------------------------------------------------------ page allocator
struct OilPages { std::vector<int32_t> free_list; std::vector<int32_t> refs; };

extern "C" {

OilPages* oil_pages_create(int32_t n) {
  auto* p = new OilPages;
  p->refs.assign(n, 0);
  for (int32_t i = n - 1; i >= 0; --i) p->free_list.push_back(i);
  return p;
}
void oil_pages_free(OilPages* p) { delete p; }
int32_t oil_pages_alloc(OilPages* p) {
  if (p->free_list.empty()) return -1;
  const int32_t id = p->free_list.back(); p->free_list.pop_back(); p->refs[id] = 1; return id;
}
void oil_pages_retain(OilPages* p, int32_t page) { if (page >= 0 && page < (int32_t)p->refs.size()) p->refs[page]++; }
void oil_pages_release(OilPages* p, int32_t page) {
  if (page < 0 || page >= (int32_t)p->refs.size() || p->refs[page] <= 0) return;
  if (--p->refs[page] == 0) p->free_list.push_back(page);
}
int32_t oil_pages_used(const OilPages* p) { return (int32_t)(p->refs.size() - p->free_list.size()); }

}  // extern "C"
