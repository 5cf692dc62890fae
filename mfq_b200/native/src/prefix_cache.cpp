// Content-addressed KV block store.
//
// A prompt is cut into blocks of `block_tokens` tokens; block i is named by
//   key[i] = SHA-256(key[i-1] || token ids of block i || salt)        (key[-1] = 32 zero bytes)
// so a key identifies the whole prefix that ends with the block, and two requests that share a prefix share keys.
// Blocks live in a RAM tier (LRU by byte budget) and, when a directory is given, in a file tier (one file per key,
// written behind by a worker thread, evicted oldest-first by byte budget).  Pinned entries are never evicted.
// Reference counterpart: cpp_runtime/core/src/mfq_paged_prefix_cache.cpp (hot tier + SSD files, async writes,
// pin/unpin, budgets).
#include "common.h"
#include "mfq_core.h"

#include <array>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <dirent.h>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <sys/stat.h>
#include <unistd.h>

namespace {
using mfqn::fail;
using Key = std::array<uint8_t, 32>;

// ---- SHA-256 (FIPS 180-4) -------------------------------------------------------------------------------------
struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t total = 0;
  size_t fill = 0;
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(h, init, sizeof h);
  }
  static uint32_t rotr(uint32_t x, int n) { return x >> n | x << (32 - n); }
  void block(const uint8_t* p) {
    static const uint32_t k[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
        0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
        0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
        0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
        0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
        0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
        0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = uint32_t(p[4 * i]) << 24 | uint32_t(p[4 * i + 1]) << 16 | uint32_t(p[4 * i + 2]) << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + k[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const void* data, size_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    total += n;
    while (n) {
      const size_t take = std::min(n, 64 - fill);
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  Key finish() {
    const uint64_t bits = total * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    uint8_t len[8];
    for (int i = 0; i < 8; ++i) len[i] = uint8_t(bits >> (56 - 8 * i));
    update(len, 8);
    Key out;
    for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) out[4 * i + j] = uint8_t(h[i] >> (24 - 8 * j));
    return out;
  }
};

std::string hex(const Key& k) {
  static const char* d = "0123456789abcdef";
  std::string s(64, '0');
  for (int i = 0; i < 32; ++i) { s[2 * i] = d[k[i] >> 4]; s[2 * i + 1] = d[k[i] & 15]; }
  return s;
}

struct Entry {
  std::shared_ptr<std::vector<uint8_t>> data;  // null when only on disk
  int64_t nbytes = 0;
  int pins = 0;
  bool on_disk = false;
  std::list<Key>::iterator lru;
  bool in_lru = false;
};

struct Cache {
  std::string dir;
  int64_t ram_budget, disk_budget;
  int block_tokens;
  std::mutex mu;
  std::map<Key, Entry> entries;
  std::list<Key> lru;        // RAM tier, most recent at the back
  std::deque<Key> disk_fifo; // file tier, oldest at the front
  int64_t ram_bytes = 0, disk_bytes = 0, hits_ram = 0, hits_disk = 0, misses = 0, evictions = 0;
  // write-behind
  std::deque<std::pair<Key, std::shared_ptr<std::vector<uint8_t>>>> pending;
  std::condition_variable cv, idle_cv;
  bool stop = false;
  int in_flight = 0;
  std::thread writer;

  std::string path_of(const Key& k) const { return dir + "/" + hex(k) + ".kv"; }

  void touch(Entry& e, const Key& k) {
    if (e.in_lru) lru.erase(e.lru);
    lru.push_back(k);
    e.lru = std::prev(lru.end());
    e.in_lru = true;
  }

  void evict_ram_locked() {
    auto it = lru.begin();
    while (ram_bytes > ram_budget && it != lru.end()) {
      auto cur = it++;
      Entry& e = entries[*cur];
      if (e.pins > 0) continue;
      ram_bytes -= e.nbytes;
      e.data.reset();
      e.in_lru = false;
      ++evictions;
      const Key k = *cur;
      lru.erase(cur);
      if (!e.on_disk && !is_pending_locked(k)) entries.erase(k);
    }
  }

  bool is_pending_locked(const Key& k) const {
    for (auto& p : pending) if (p.first == k) return true;
    return false;
  }

  void evict_disk_locked() {
    size_t budget = disk_fifo.size();  // every entry is looked at once at most: all-pinned tiers cannot spin
    while (disk_bytes > disk_budget && !disk_fifo.empty() && budget-- > 0) {
      const Key k = disk_fifo.front();
      disk_fifo.pop_front();
      auto it = entries.find(k);
      if (it == entries.end() || !it->second.on_disk) continue;
      if (it->second.pins > 0) { disk_fifo.push_back(k); continue; }
      unlink(path_of(k).c_str());
      disk_bytes -= it->second.nbytes;
      it->second.on_disk = false;
      ++evictions;
      if (!it->second.data) entries.erase(it);
    }
  }

  void writer_loop() {
    std::unique_lock<std::mutex> lk(mu);
    while (true) {
      cv.wait(lk, [&] { return stop || !pending.empty(); });
      if (pending.empty()) { if (stop) return; continue; }
      auto job = pending.front();
      ++in_flight;
      lk.unlock();
      const std::string path = path_of(job.first), tmp = path + ".tmp";
      bool ok = false;
      if (FILE* f = fopen(tmp.c_str(), "wb")) {
        ok = fwrite(job.second->data(), 1, job.second->size(), f) == job.second->size();
        ok = fclose(f) == 0 && ok;
        ok = ok && rename(tmp.c_str(), path.c_str()) == 0;
        if (!ok) unlink(tmp.c_str());
      }
      lk.lock();
      pending.pop_front();
      --in_flight;
      auto it = entries.find(job.first);
      if (ok && it != entries.end() && !it->second.on_disk) {
        it->second.on_disk = true;
        disk_bytes += it->second.nbytes;
        disk_fifo.push_back(job.first);
        evict_disk_locked();
      } else if (ok && it == entries.end()) {
        unlink(path.c_str());
      }
      if (pending.empty() && in_flight == 0) idle_cv.notify_all();
    }
  }
};

Key to_key(const uint8_t* p) { Key k; memcpy(k.data(), p, 32); return k; }
}  // namespace

extern "C" {

void* mfq_prefix_open(const char* dir, int64_t ram_budget, int64_t disk_budget, int block_tokens) {
  if (block_tokens <= 0 || ram_budget < 0) { fail(-1, "bad prefix cache parameters"); return nullptr; }
  auto c = new Cache();
  c->dir = dir ? dir : "";
  c->ram_budget = ram_budget;
  c->disk_budget = c->dir.empty() ? 0 : disk_budget;
  c->block_tokens = block_tokens;
  if (!c->dir.empty()) {
    mkdir(c->dir.c_str(), 0755);
    // adopt blocks left by an earlier process
    if (DIR* d = opendir(c->dir.c_str())) {
      while (dirent* ent = readdir(d)) {
        const std::string name = ent->d_name;
        if (name.size() != 67 || name.compare(64, 3, ".kv") != 0) continue;
        Key k;
        bool ok = true;
        for (int i = 0; i < 32 && ok; ++i) {
          auto nib = [&](char ch) { return ch >= '0' && ch <= '9' ? ch - '0' : ch >= 'a' && ch <= 'f' ? ch - 'a' + 10 : (ok = false, 0); };
          k[i] = uint8_t(nib(name[2 * i]) << 4 | nib(name[2 * i + 1]));
        }
        struct stat st;
        if (!ok || stat((c->dir + "/" + name).c_str(), &st) != 0) continue;
        Entry e;
        e.nbytes = st.st_size;
        e.on_disk = true;
        c->entries[k] = e;
        c->disk_fifo.push_back(k);
        c->disk_bytes += st.st_size;
      }
      closedir(d);
    }
    c->writer = std::thread([c] { c->writer_loop(); });
  }
  return c;
}

void mfq_prefix_close(void* cache) {
  auto* c = static_cast<Cache*>(cache);
  if (c->writer.joinable()) {
    { std::lock_guard<std::mutex> lk(c->mu); c->stop = true; }
    c->cv.notify_all();
    c->writer.join();
  }
  delete c;
}

int mfq_prefix_keys(void* cache, const int32_t* tokens, int64_t n_tokens, const char* salt, uint8_t* keys_out) {
  auto* c = static_cast<Cache*>(cache);
  const int64_t blocks = n_tokens / c->block_tokens;
  Key prev{};
  for (int64_t b = 0; b < blocks; ++b) {
    Sha256 h;
    h.update(prev.data(), 32);
    h.update(tokens + b * c->block_tokens, size_t(c->block_tokens) * 4);
    if (salt) h.update(salt, strlen(salt));
    prev = h.finish();
    memcpy(keys_out + 32 * b, prev.data(), 32);
  }
  return int(blocks);
}

int mfq_prefix_put(void* cache, const uint8_t* key, const void* data, int64_t nbytes) {
  auto* c = static_cast<Cache*>(cache);
  const Key k = to_key(key);
  auto buf = std::make_shared<std::vector<uint8_t>>(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + nbytes);
  std::lock_guard<std::mutex> lk(c->mu);
  Entry& e = c->entries[k];
  if (e.data) return 0;  // already hot
  const bool had_disk = e.on_disk;
  e.data = buf;
  e.nbytes = nbytes;
  c->ram_bytes += nbytes;
  c->touch(e, k);
  if (!c->dir.empty() && !had_disk && c->disk_budget > 0) {
    c->pending.emplace_back(k, buf);
    c->cv.notify_one();
  }
  c->evict_ram_locked();
  return 0;
}

int64_t mfq_prefix_get(void* cache, const uint8_t* key, void* dst, int64_t capacity) {
  auto* c = static_cast<Cache*>(cache);
  const Key k = to_key(key);
  std::unique_lock<std::mutex> lk(c->mu);
  auto it = c->entries.find(k);
  if (it == c->entries.end()) { ++c->misses; return -1; }
  Entry& e = it->second;
  if (e.nbytes > capacity) return fail(-2, "destination too small for the block");
  if (e.data) {
    memcpy(dst, e.data->data(), size_t(e.nbytes));
    c->touch(e, k);
    ++c->hits_ram;
    return e.nbytes;
  }
  if (!e.on_disk) { ++c->misses; return -1; }
  const std::string path = c->path_of(k);
  const int64_t n = e.nbytes;
  lk.unlock();
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) { lk.lock(); ++c->misses; return -1; }
  auto buf = std::make_shared<std::vector<uint8_t>>(size_t(n));
  const bool ok = fread(buf->data(), 1, size_t(n), f) == size_t(n);
  fclose(f);
  lk.lock();
  if (!ok) { ++c->misses; return -1; }
  memcpy(dst, buf->data(), size_t(n));
  ++c->hits_disk;
  auto it2 = c->entries.find(k);
  if (it2 != c->entries.end() && !it2->second.data) {  // promote to the hot tier
    it2->second.data = buf;
    c->ram_bytes += n;
    c->touch(it2->second, k);
    c->evict_ram_locked();
  }
  return n;
}

int mfq_prefix_match(void* cache, const uint8_t* keys, int n_keys) {
  auto* c = static_cast<Cache*>(cache);
  std::lock_guard<std::mutex> lk(c->mu);
  int n = 0;
  while (n < n_keys) {
    auto it = c->entries.find(to_key(keys + 32 * n));
    if (it == c->entries.end() || (!it->second.data && !it->second.on_disk)) break;
    ++n;
  }
  return n;
}

int mfq_prefix_pin(void* cache, const uint8_t* key, int delta) {
  auto* c = static_cast<Cache*>(cache);
  std::lock_guard<std::mutex> lk(c->mu);
  auto it = c->entries.find(to_key(key));
  if (it == c->entries.end()) return fail(-1, "no such block");
  it->second.pins = std::max(0, it->second.pins + delta);
  if (it->second.pins == 0) { c->evict_ram_locked(); c->evict_disk_locked(); }
  return 0;
}

int mfq_prefix_flush(void* cache) {
  auto* c = static_cast<Cache*>(cache);
  std::unique_lock<std::mutex> lk(c->mu);
  c->idle_cv.wait(lk, [&] { return c->pending.empty() && c->in_flight == 0; });
  return 0;
}

int mfq_prefix_stats(void* cache, int64_t* out8) {
  auto* c = static_cast<Cache*>(cache);
  std::lock_guard<std::mutex> lk(c->mu);
  int64_t ram_entries = 0, disk_entries = 0;
  for (auto& kv : c->entries) { ram_entries += kv.second.data != nullptr; disk_entries += kv.second.on_disk; }
  const int64_t v[8] = {c->ram_bytes, c->disk_bytes, ram_entries, disk_entries, c->hits_ram, c->hits_disk, c->misses, c->evictions};
  memcpy(out8, v, sizeof v);
  return 0;
}
}
