// Memory-mapped `.mfq` reader.
//
// Layout (little endian): "MFQ1", u32 version, str arch, [version >= 2: u32 n, n x (str key, str json)],
// u32 n_tensors, n x (str name, str dtype, u64 nbytes), then the blobs back to back (str = u32 length + bytes).
// A shard set `stem-00001-of-0000N.mfq` is opened as one store; records keep their shard index.
// Reference counterpart: cpp_runtime/core/src/mfq_model_source.cpp (parser) and file_range_reader.cpp (range reads).
#include "common.h"
#include "mfq_core.h"

#include <cstring>
#include <exception>
#include <memory>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <unordered_map>
#include <vector>

namespace {
using mfqn::fail;

struct Mapping {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t size = 0;
};

struct Record {
  std::string name, dtype;
  int64_t offset = 0, nbytes = 0;
  int file = 0;
};

struct Store {
  std::vector<Mapping> files;
  std::vector<Record> records;
  std::unordered_map<std::string, int64_t> index;
  int version = 0;
  std::string arch;
  std::vector<std::pair<std::string, std::string>> extra;
  ~Store() {
    for (auto& m : files) {
      if (m.base) munmap(const_cast<uint8_t*>(m.base), m.size);
      if (m.fd >= 0) close(m.fd);
    }
  }
};

struct Cursor {
  const uint8_t* p;
  size_t left;
  bool ok = true;
  template <typename T> T get() {
    T v{};
    if (left < sizeof(T)) { ok = false; return v; }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    left -= sizeof(T);
    return v;
  }
  std::string str() {
    const uint32_t n = get<uint32_t>();
    if (!ok || left < n) { ok = false; return {}; }
    std::string s(reinterpret_cast<const char*>(p), n);
    p += n;
    left -= n;
    return s;
  }
};

bool map_file(const std::string& path, Mapping& m) {
  m.fd = open(path.c_str(), O_RDONLY);
  if (m.fd < 0) return false;
  struct stat st;
  if (fstat(m.fd, &st) != 0 || st.st_size < 12) return false;
  m.size = size_t(st.st_size);
  void* p = mmap(nullptr, m.size, PROT_READ, MAP_SHARED, m.fd, 0);
  if (p == MAP_FAILED) return false;
  m.base = static_cast<const uint8_t*>(p);
  return true;
}

// "stem-00003-of-00007.mfq" -> (stem, 3, 7)
bool split_shard_name(const std::string& path, std::string& stem, int& index, int& count) {
  const size_t n = path.size();
  if (n < 4 + 19 || path.compare(n - 4, 4, ".mfq") != 0) return false;
  const size_t tail = n - 4 - 15;  // "-00003-of-00007"
  const std::string t = path.substr(tail, 15);
  if (t[0] != '-' || t.compare(6, 4, "-of-") != 0) return false;
  for (int i : {1, 2, 3, 4, 5, 10, 11, 12, 13, 14})
    if (t[i] < '0' || t[i] > '9') return false;
  stem = path.substr(0, tail);
  index = atoi(t.substr(1, 5).c_str());
  count = atoi(t.substr(10, 5).c_str());
  return count >= 1 && index >= 1 && index <= count;
}

int parse_into(Store& s, int file_index, bool first) {
  const Mapping& m = s.files[file_index];
  Cursor c{m.base, m.size};
  if (memcmp(c.p, "MFQ1", 4) != 0) return fail(-2, "shard %d: bad magic", file_index);
  c.p += 4;
  c.left -= 4;
  const uint32_t version = c.get<uint32_t>();
  const std::string arch = c.str();
  std::vector<std::pair<std::string, std::string>> extra;
  if (version >= 2) {
    const uint32_t n = c.get<uint32_t>();
    for (uint32_t i = 0; i < n && c.ok; ++i) {
      std::string k = c.str(), v = c.str();
      extra.emplace_back(std::move(k), std::move(v));
    }
  }
  const uint32_t n_tensors = c.get<uint32_t>();
  if (!c.ok) return fail(-2, "shard %d: truncated header", file_index);
  // sizes in the file are not trusted: a record takes at least 16 bytes of table (two length words + the blob size)
  if (uint64_t(n_tensors) > uint64_t(c.left) / 16) return fail(-2, "shard %d: tensor count exceeds the file size", file_index);
  std::vector<Record> recs;
  recs.reserve(n_tensors);
  for (uint32_t i = 0; i < n_tensors; ++i) {
    Record r;
    r.name = c.str();
    r.dtype = c.str();
    r.nbytes = int64_t(c.get<uint64_t>());
    r.file = file_index;
    if (!c.ok || r.nbytes < 0) return fail(-2, "shard %d: truncated record table", file_index);
    recs.push_back(std::move(r));
  }
  int64_t off = int64_t(c.p - m.base);
  for (auto& r : recs) {
    // checked per record, against what is left, so that a crafted size cannot wrap the running offset
    if (uint64_t(r.nbytes) > uint64_t(m.size) - uint64_t(off))
      return fail(-2, "shard %d: blobs run past the end of the file", file_index);
    r.offset = off;
    off += r.nbytes;
  }
  if (first) {
    s.version = int(version);
    s.arch = arch;
    s.extra = std::move(extra);
  }
  for (auto& r : recs) {
    if (s.index.count(r.name)) return fail(-2, "tensor '%s' appears twice", r.name.c_str());
    s.index[r.name] = int64_t(s.records.size());
    s.records.push_back(std::move(r));
  }
  return 0;
}
}  // namespace

extern "C" {

const char* mfq_last_error() { return mfqn::error_slot().c_str(); }

void* mfq_store_open(const char* path) try {
  std::unique_ptr<Store> s(new Store());
  std::string stem;
  int index = 0, count = 0;
  std::vector<std::string> paths;
  if (split_shard_name(path, stem, index, count)) {
    char buf[32];
    for (int i = 1; i <= count; ++i) {
      snprintf(buf, sizeof buf, "-%05d-of-%05d.mfq", i, count);
      paths.push_back(stem + buf);
    }
  } else {
    paths.emplace_back(path);
  }
  for (size_t i = 0; i < paths.size(); ++i) {
    s->files.emplace_back();
    if (!map_file(paths[i], s->files.back())) {
      fail(-1, "cannot map '%s'", paths[i].c_str());
      return nullptr;
    }
    if (parse_into(*s, int(i), i == 0) != 0) {
      return nullptr;
    }
  }
  return s.release();
} catch (const std::exception& e) {  // nothing may unwind through the C boundary
  fail(-3, "opening the container failed: %s", e.what());
  return nullptr;
}

void mfq_store_close(void* store) { delete static_cast<Store*>(store); }
int mfq_store_version(void* store) { return static_cast<Store*>(store)->version; }
const char* mfq_store_arch(void* store) { return static_cast<Store*>(store)->arch.c_str(); }
int mfq_store_extra_count(void* store) { return int(static_cast<Store*>(store)->extra.size()); }
const char* mfq_store_extra_key(void* store, int i) { return static_cast<Store*>(store)->extra[i].first.c_str(); }
const char* mfq_store_extra_json(void* store, int i) { return static_cast<Store*>(store)->extra[i].second.c_str(); }
int64_t mfq_store_tensor_count(void* store) { return int64_t(static_cast<Store*>(store)->records.size()); }
const char* mfq_store_tensor_name(void* store, int64_t i) { return static_cast<Store*>(store)->records[i].name.c_str(); }
const char* mfq_store_tensor_dtype(void* store, int64_t i) { return static_cast<Store*>(store)->records[i].dtype.c_str(); }
int64_t mfq_store_tensor_nbytes(void* store, int64_t i) { return static_cast<Store*>(store)->records[i].nbytes; }
int mfq_store_tensor_file(void* store, int64_t i) { return static_cast<Store*>(store)->records[i].file; }

int64_t mfq_store_find(void* store, const char* name) {
  auto& idx = static_cast<Store*>(store)->index;
  auto it = idx.find(name);
  return it == idx.end() ? -1 : it->second;
}

const void* mfq_store_tensor_data(void* store, int64_t i) {
  auto* s = static_cast<Store*>(store);
  const Record& r = s->records[i];
  return s->files[r.file].base + r.offset;
}

int mfq_store_read(void* store, int64_t i, int64_t offset, int64_t nbytes, void* dst, int threads, int drop_cache) {
  auto* s = static_cast<Store*>(store);
  if (i < 0 || i >= int64_t(s->records.size())) return fail(-1, "tensor index out of range");
  const Record& r = s->records[i];
  if (offset < 0 || nbytes < 0 || offset + nbytes > r.nbytes) return fail(-1, "range outside the blob of '%s'", r.name.c_str());
  const uint8_t* src = s->files[r.file].base + r.offset + offset;
  constexpr int64_t kChunk = 4 << 20;
  const int64_t chunks = (nbytes + kChunk - 1) / kChunk;
  mfqn::parallel_for(chunks, threads, [&](int64_t b, int64_t e) {
    for (int64_t c = b; c < e; ++c) {
      const int64_t o = c * kChunk, n = std::min(kChunk, nbytes - o);
      memcpy(static_cast<uint8_t*>(dst) + o, src + o, size_t(n));
    }
  });
  if (drop_cache) {
    const long page = sysconf(_SC_PAGESIZE);
    const uintptr_t a = reinterpret_cast<uintptr_t>(src) & ~uintptr_t(page - 1);
    madvise(reinterpret_cast<void*>(a), size_t(reinterpret_cast<uintptr_t>(src) + nbytes - a), MADV_DONTNEED);
  }
  return 0;
}
}
