// Error reporting and the host-side index helpers of include/thb200.h.
#include "thb_internal.h"

#include <algorithm>
#include <climits>
#include <cstdarg>
#include <cstdio>
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace thb {

static thread_local std::string g_last_error;

int fail(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return 1;
}

int fail_cuda(cudaError_t e, const char* what) {
  return fail("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

int64_t num_elements(const thb200_tensor& t) {
  if (t.ndim == 0) return 0;
  int64_t n = 1;
  for (int i = 0; i < t.ndim; ++i) n *= t.size[i];
  return n;
}

// Dimension collapsing, following TensorInfo<IndexType>::TensorInfo
// (reference src/lib/THClReduceApplyUtils.h:68-170): walk from the innermost
// dimension outwards, skip size-1 dims (the reduce dim counts as size 1), and
// fold an outer dim into the current run when its stride continues the run.
bool collapse(int ndim, const int64_t* size, const int64_t* stride, int reduce_dim, Collapsed* out) {
  if (ndim < 0 || ndim > THB200_MAX_DIMS || reduce_dim >= ndim) return false;
  int64_t rs[THB200_MAX_DIMS], rst[THB200_MAX_DIMS];  // runs, innermost first
  int nruns = 0;
  for (int i = ndim - 1; i >= 0; --i) {
    int64_t sz = (i == reduce_dim) ? 1 : size[i];
    if (sz == 1) continue;
    if (nruns > 0 && stride[i] == rs[nruns - 1] * rst[nruns - 1]) {
      rs[nruns - 1] *= sz;
    } else {
      rs[nruns] = sz;
      rst[nruns] = stride[i];
      ++nruns;
    }
  }
  if (nruns == 0) {  // every dim has size 1: a single point
    out->dims = 1;
    out->size[0] = 1;
    out->stride[0] = 1;
    return true;
  }
  out->dims = nruns;
  for (int i = 0; i < nruns; ++i) {
    out->size[i] = rs[nruns - 1 - i];
    out->stride[i] = rst[nruns - 1 - i];
  }
  return true;
}

// Largest reachable offset and the element count both below UINT_MAX
// (reference src/lib/THClReduceApplyUtils.cpp:9-30).
bool can_use_32bit(int ndim, const int64_t* size, const int64_t* stride) {
  int64_t n = 1;
  for (int i = 0; i < ndim; ++i) n *= size[i];
  if (ndim == 0) n = 0;
  if (n >= (int64_t)UINT_MAX) return false;
  int64_t offset = 0;
  for (int i = ndim - 1; i >= 0; --i) {
    if (size[i] > 0) offset += (size[i] - 1) * stride[i];
  }
  return offset < (int64_t)UINT_MAX;
}

int sm_count() {
  static std::mutex mu;
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- which end of its operands the last streaming kernel left in L2 ----------------------------------
// A kernel that streams through operands larger than L2 leaves the part it touched last in L2 (dirty, if it
// wrote it). The next kernel over the same memory saves that much HBM traffic, and the write-back of lines
// it overwrites, when it starts at that end. Per device, the last kernel's final window of every operand is
// remembered; a contiguous apply walks its batches downwards when more of the remembered bytes lie in the
// last window of its operands than in the first. Only the order in time changes, never a result.
namespace {
struct HotState {
  uintptr_t lo[3] = {0, 0, 0}, hi[3] = {0, 0, 0};
  int count = 0;
  size_t l2_bytes = 0;
};
std::mutex g_hot_mu;
HotState g_hot[64];

HotState* hot_state() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  HotState* h = &g_hot[dev];
  if (h->l2_bytes == 0) {
    int v = 0;
    h->l2_bytes = (cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev) == cudaSuccess && v > 0) ? (size_t)v : 1;
  }
  return h;
}
size_t overlap(uintptr_t a0, uintptr_t a1, uintptr_t b0, uintptr_t b1) {
  const uintptr_t lo = a0 > b0 ? a0 : b0, hi = a1 < b1 ? a1 : b1;
  return hi > lo ? (size_t)(hi - lo) : 0;
}
}  // namespace

bool stream_prefers_descending(const void* const* ptrs, int n, size_t bytes) {
  std::lock_guard<std::mutex> lock(g_hot_mu);
  HotState* h = hot_state();
  if (!h || n < 1 || n > 3) return false;
  const size_t window = h->l2_bytes * 3 / 4 / (size_t)n;
  if (bytes <= 2 * window) return false;  // (nearly) all of it can be in L2: the order does not matter
  size_t first = 0, last = 0;
  for (int i = 0; i < n; ++i) {
    const uintptr_t p = (uintptr_t)ptrs[i];
    for (int k = 0; k < h->count; ++k) {
      first += overlap(p, p + window, h->lo[k], h->hi[k]);
      last += overlap(p + bytes - window, p + bytes, h->lo[k], h->hi[k]);
    }
  }
  return last > first;
}

void stream_note_end(const void* const* ptrs, int n, size_t bytes, bool descending) {
  std::lock_guard<std::mutex> lock(g_hot_mu);
  HotState* h = hot_state();
  if (!h || n < 1 || n > 3) return;
  size_t window = h->l2_bytes * 3 / 4 / (size_t)n;
  if (window > bytes) window = bytes;
  h->count = n;
  for (int i = 0; i < n; ++i) {
    const uintptr_t p = (uintptr_t)ptrs[i];
    h->lo[i] = descending ? p : p + bytes - window;
    h->hi[i] = descending ? p + window : p + bytes;
  }
}

}  // namespace thb

extern "C" {

const char* thb200_last_error(void) { return thb::g_last_error.c_str(); }

int thb200_collapse_dims(int ndim, const int64_t* size, const int64_t* stride, int reduce_dim,
                         int64_t* out_size, int64_t* out_stride) {
  thb::Collapsed c;
  if (!thb::collapse(ndim, size, stride, reduce_dim, &c)) {
    thb::fail("collapse: bad arguments (ndim=%d, reduce_dim=%d)", ndim, reduce_dim);
    return -1;
  }
  for (int i = 0; i < c.dims; ++i) {
    out_size[i] = c.size[i];
    out_stride[i] = c.stride[i];
  }
  return c.dims;
}

int thb200_can_use_32bit_index(int ndim, const int64_t* size, const int64_t* stride) {
  return thb::can_use_32bit(ndim, size, stride) ? 1 : 0;
}

int thb200_overlapping_indices(int ndim, const int64_t* size, const int64_t* stride) {
  // Dims of size > 1 sorted by ascending stride; the view overlaps itself when
  // the smallest stride is < 1 or when a dim does not clear the extent of the
  // next smaller one (reference src/lib/THClReduceApplyUtils.cpp:69-121).
  std::pair<int64_t, int64_t> d[THB200_MAX_DIMS];  // (stride, size)
  int k = 0;
  for (int i = 0; i < ndim && i < THB200_MAX_DIMS; ++i)
    if (size[i] > 1) d[k++] = std::make_pair(stride[i], size[i]);
  if (k == 0) return 0;
  std::sort(d, d + k);
  if (d[0].first < 1) return 1;
  for (int i = 1; i < k; ++i)
    if (d[i].first < d[i - 1].first * d[i - 1].second) return 1;
  return 0;
}

}  // extern "C"

// ---- per-call device timing ---------------------------------------------------
// The thin equivalent of cltorch.setProfiling / dumpProfiling and setEnableTiming / dumpTimings
// (reference src/init.cpp:130-178): device time per entry point, from CUDA events on the call's stream.
namespace thb {
namespace {
struct Pending { const char* name; cudaEvent_t start, stop; };
struct Bucket { long calls = 0; double ms = 0.0; };
std::mutex g_timing_mu;
std::atomic<bool> g_timing_on{false};
std::vector<Pending> g_pending;
std::vector<cudaEvent_t> g_free_events;
std::map<std::string, Bucket> g_buckets;

cudaEvent_t take_event() {
  if (!g_free_events.empty()) { cudaEvent_t e = g_free_events.back(); g_free_events.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  return e;
}
// resolves every finished pair; with `wait`, waits for the unfinished ones too
void drain(bool wait) {
  std::vector<Pending> keep;
  for (const Pending& p : g_pending) {
    cudaError_t q = wait ? cudaEventSynchronize(p.stop) : cudaEventQuery(p.stop);
    if (q == cudaErrorNotReady) { keep.push_back(p); continue; }
    float ms = 0.f;
    if (q == cudaSuccess && cudaEventElapsedTime(&ms, p.start, p.stop) == cudaSuccess) {
      Bucket& b = g_buckets[p.name];
      b.calls += 1;
      b.ms += ms;
    } else {
      cudaGetLastError();
    }
    g_free_events.push_back(p.start);
    g_free_events.push_back(p.stop);
  }
  g_pending.swap(keep);
}
}  // namespace

CallTimer::CallTimer(void* stream, const char* name) {
  if (!g_timing_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lock(g_timing_mu);
  start_ = take_event();
  stop_ = take_event();
  if (!start_ || !stop_) { start_ = stop_ = nullptr; return; }
  stream_ = (cudaStream_t)stream;
  name_ = name;
  cudaEventRecord(start_, stream_);
}
CallTimer::~CallTimer() {
  if (!start_) return;
  cudaEventRecord(stop_, stream_);
  std::lock_guard<std::mutex> lock(g_timing_mu);
  g_pending.push_back(Pending{name_, start_, stop_});
  if (g_pending.size() > 4096) drain(false);
}
}  // namespace thb

extern "C" {

void thb200_timing_enable(int on) { thb::g_timing_on.store(on != 0, std::memory_order_relaxed); }

void thb200_timing_reset(void) {
  std::lock_guard<std::mutex> lock(thb::g_timing_mu);
  thb::drain(true);
  thb::g_buckets.clear();
}

size_t thb200_timing_report(char* buf, size_t capacity) {
  std::lock_guard<std::mutex> lock(thb::g_timing_mu);
  thb::drain(true);
  std::string out;
  char line[256];
  for (const auto& kv : thb::g_buckets) {
    snprintf(line, sizeof line, "%s %ld %.6f\n", kv.first.c_str(), kv.second.calls, kv.second.ms);
    out += line;
  }
  if (buf && capacity > 0) {
    size_t n = out.size() < capacity - 1 ? out.size() : capacity - 1;
    memcpy(buf, out.data(), n);
    buf[n] = 0;
  }
  return out.size() + 1;
}

}  // extern "C"
