// Shared helpers of the host runtime library: thread-local error text and a small fork-join helper.
#pragma once
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <functional>
#include <string>
#include <thread>
#include <vector>

namespace mfqn {

inline std::string& error_slot() {
  thread_local std::string s;
  return s;
}

inline int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  error_slot() = buf;
  return code;
}

// Runs fn(begin, end) over [0, n) split into at most `threads` contiguous chunks (inline when threads <= 1).
inline void parallel_for(int64_t n, int threads, const std::function<void(int64_t, int64_t)>& fn) {
  if (n <= 0) return;
  const int64_t t = std::max<int64_t>(1, std::min<int64_t>(threads, n));
  if (t == 1) { fn(0, n); return; }
  std::vector<std::thread> pool;
  const int64_t per = (n + t - 1) / t;
  for (int64_t i = 0; i < t; ++i) {
    const int64_t b = i * per, e = std::min(n, b + per);
    if (b >= e) break;
    pool.emplace_back(fn, b, e);
  }
  for (auto& th : pool) th.join();
}

}  // namespace mfqn
