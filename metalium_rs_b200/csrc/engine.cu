// The engine behind include/b200tt.h: host-side state and routing for one GPU.
//
// It plays the part of an `impl burn_tt::Engine` (crates/burn-tt/src/server.rs:42-786)
// with the reference's `Session`, GDDR allocator, L1 planner and data movers
// (crates/tt-kernels/src/session.rs:824) replaced by
//   - a device-memory pool (cached blocks, reuse in stream order),
//   - a buffer table `id -> {ptr, rows, cols, elem}` with views that keep their parent alive,
//   - one CUDA stream on which every op is launched in call order,
//   - a device error word read at the waits (an index out of its table, a division by
//     zero), so a failed op never traps the GPU.
// No op falls back to host arithmetic: what the kernels cannot do is refused.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <cmath>

#include <algorithm>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/b200tt.h"
#include "kernels.h"
#include "kinds.h"

using namespace b200;

namespace {

// Text of failures that belong to no engine (a refused create, an engine-less entry point); calls that
// take no engine may come from any thread, so it is guarded.
std::mutex g_global_lock;
std::string g_create_error;
void set_create_error(const std::string& text) { std::lock_guard<std::mutex> hold(g_global_lock); g_create_error = text; }

struct Buf {
  void* ptr = nullptr;
  uint64_t rows = 0, cols = 0;
  int elem = B200_F32;
  uint64_t bytes = 0;       // bytes of the pool block (0 for views / adopted memory)
  b200_buffer parent = 0;   // view of another buffer
  int views = 0;            // live views of this buffer
  bool freed = false;       // free() called while views are alive
  bool adopted = false;
};

inline uint64_t elem_bytes(int elem) { return elem == B200_BF16 ? 2 : 4; }
// Bytes a [rows, cols] buffer of `elem` holds: a BFP8 matrix is a datum byte an element and an exponent byte
// for every sixteen of a row (csrc/k_bfp.cu).
inline uint64_t buffer_bytes(uint64_t rows, uint64_t cols, int elem) {
  return elem == B200_BFP8 ? rows * cols + rows * cols / 16 : rows * cols * elem_bytes(elem);
}

}  // namespace

struct b200_engine {
  int device = 0;
  b200_config cfg{};
  cudaStream_t stream = nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  int* d_err = nullptr;
  long long wait_limit_word = 0;   // host copy of the limit kept behind the device error word
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;   // b200_matmul_host_bf16's copy streams
  int matmul_sm_limit = 0;   // b200_set_matmul_sm_limit
  int* h_err = nullptr;  // pinned
  std::string last_error;
  uint64_t oom[3] = {0, 0, 0};
  int sticky = 0;  // first asynchronous failure, reported at every later wait
  std::string sticky_text;
  std::string label;
  const char* matmul_path = "none";
  const char* decode_form = "none";
  b200_traffic traffic{};
  uint64_t next_id = 1;
  uint64_t alloc_calls = 0;
  std::unordered_map<b200_buffer, Buf> bufs;
  std::multimap<uint64_t, void*> cache;  // free blocks by size
  float* full_scratch = nullptr;
  // Traces (CUDA graphs): the counterpart of the reference's begin_trace / end_trace / run_trace
  // (crates/burn-tt/src/server.rs:591-660).  While one is captured, every block the ops take is
  // owned by the trace: a replay writes the same addresses, so they must not go back to the pool
  // before the trace is released.
  struct Trace {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<std::pair<void*, uint64_t>> blocks;   // every block the capture took
    std::vector<void*> pinned;                        // host copies of block lists the graph re-uploads
    uint64_t launches = 0;
    std::vector<std::pair<std::string, uint64_t>> ops;   // the captured ops in order: (label, kernels)
  };
  bool capturing = false;
  Trace cur;                                          // the trace being captured
  std::multimap<uint64_t, void*> cur_free;            // its blocks free for reuse inside the capture
  std::unordered_map<void*, uint64_t> cur_owned;      // ptr -> size of blocks the capture owns
  std::unordered_map<uint64_t, Trace> traces;
  uint64_t next_trace = 1;
  // Per-op device time (the profile mode, crates/burn-tt/src/profile.rs:1-48): while it is on, every
  // `set_op_label` records an event on the stream, so the device time between two labels is charged to the
  // first one -- the server labels each job before it runs it (server.rs:2370 `timed_job`).
  struct Mark { std::string label; cudaEvent_t at = nullptr; uint64_t launches = 0; };
  bool profiling = false;
  std::vector<Mark> marks;                 // marks[i] opens op i; the next mark (or `prof_end`) closes it
  cudaEvent_t prof_end = nullptr;
  struct Stat { uint64_t calls = 0, launches = 0; double ms = 0; };
  std::vector<std::pair<std::string, Stat>> prof_table;   // in order of first appearance
  void drop_marks() {
    for (auto& m : marks) if (m.at) cudaEventDestroy(m.at);
    marks.clear();
    if (prof_end) { cudaEventDestroy(prof_end); prof_end = nullptr; }
  }

  int fail(int code, const char* fmt, ...) {
    char tmp[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tmp, sizeof tmp, fmt, ap);
    va_end(ap);
    last_error = label.empty() ? std::string(tmp) : (label + ": " + tmp);
    return code;
  }
  int cuda_fail(cudaError_t e, const char* what) {
    return fail(B200_DEVICE, "%s: %s", what, cudaGetErrorString(e));
  }

  // ---- pool ---------------------------------------------------------------------
  static uint64_t round_size(uint64_t n) {
    if (n == 0) n = 1;
    if (n <= 4096) return (n + 255) & ~255ull;
    if (n <= (1ull << 20)) {
      uint64_t p = 4096;
      while (p < n) p <<= 1;
      return p;
    }
    return (n + (2ull << 20) - 1) & ~((2ull << 20) - 1);
  }
  void release_cache() {
    for (auto& kv : cache) {
      cudaFree(kv.second);
      traffic.pool_reserved -= kv.first;
    }
    cache.clear();
  }
  int alloc(uint64_t bytes, void** out, uint64_t* got) {
    ++alloc_calls;
    const uint64_t sz = round_size(bytes);
    if (cfg.fail_alloc_at > 0 && alloc_calls == (uint64_t)cfg.fail_alloc_at) {
      oom[0] = sz; oom[1] = 0; oom[2] = 0;
      return fail(B200_OUT_OF_MEMORY, "out of device memory: need %llu bytes (injected)", (unsigned long long)sz);
    }
    if (capturing) {
      auto ft = cur_free.lower_bound(sz);
      if (ft != cur_free.end() && ft->first <= sz + sz / 4) {
        *out = ft->second; *got = ft->first;
        cur_free.erase(ft);
        traffic.pool_in_use += *got;
        traffic.pool_high_water = std::max(traffic.pool_high_water, traffic.pool_in_use);
        return B200_OK;
      }
    }
    auto it = cache.lower_bound(sz);
    if (it != cache.end() && it->first <= sz + sz / 4) {
      *out = it->second;
      *got = it->first;
      cache.erase(it);
    } else {
      if (cfg.pool_limit_bytes && traffic.pool_reserved + sz > cfg.pool_limit_bytes) release_cache();
      if (cfg.pool_limit_bytes && traffic.pool_reserved + sz > cfg.pool_limit_bytes) {
        oom[0] = sz; oom[1] = cfg.pool_limit_bytes - traffic.pool_reserved; oom[2] = oom[1];
        return fail(B200_OUT_OF_MEMORY, "out of device memory: need %llu bytes, pool limit leaves %llu",
                    (unsigned long long)sz, (unsigned long long)oom[1]);
      }
      void* p = nullptr;
      cudaError_t e = cudaMalloc(&p, sz);
      if (e != cudaSuccess && !capturing) {   // a synchronise would invalidate an open capture: fail at once there
        cudaGetLastError();
        cudaStreamSynchronize(stream);
        release_cache();
        e = cudaMalloc(&p, sz);
      }
      if (e != cudaSuccess) {
        cudaGetLastError();
        size_t fr = 0, tot = 0;
        cudaMemGetInfo(&fr, &tot);
        oom[0] = sz; oom[1] = fr; oom[2] = fr;
        return fail(B200_OUT_OF_MEMORY, "out of device memory: need %llu bytes, %llu free",
                    (unsigned long long)sz, (unsigned long long)fr);
      }
      *out = p;
      *got = sz;
      traffic.pool_reserved += sz;
    }
    traffic.pool_in_use += *got;
    traffic.pool_high_water = std::max(traffic.pool_high_water, traffic.pool_in_use);
    if (capturing) { cur.blocks.emplace_back(*out, *got); cur_owned.emplace(*out, *got); }
    return B200_OK;
  }
  // Whether a block belongs to a trace (captured or being captured): such a block never
  // returns to the pool while its trace lives.
  std::unordered_set<void*> trace_ptrs;   // blocks of finished traces still alive
  bool trace_owned(void* p) const { return cur_owned.count(p) != 0 || trace_ptrs.count(p) != 0; }
  // The block returns to the cache at once: every user of it was enqueued on the one
  // stream before this call, and so is every later user.
  void release(void* p, uint64_t sz) {
    if (sz == 0) return;                 // a kept block list: the engine's, not the pool's
    traffic.pool_in_use -= sz;
    if (capturing && cur_owned.count(p)) { cur_free.emplace(sz, p); return; }
    if (trace_owned(p)) return;   // its trace keeps it
    cache.emplace(sz, p);
  }

  // ---- buffer table ------------------------------------------------------------
  int new_buffer(uint64_t rows, uint64_t cols, int elem, b200_buffer* id, Buf** out) {
    void* p = nullptr;
    uint64_t got = 0;
    const uint64_t bytes = buffer_bytes(rows, cols, elem);
    int st = alloc(bytes, &p, &got);
    if (st) return st;
    Buf b;
    b.ptr = p; b.rows = rows; b.cols = cols; b.elem = elem; b.bytes = got;
    *id = next_id++;
    auto ins = bufs.emplace(*id, b);
    if (out) *out = &ins.first->second;
    return B200_OK;
  }
  Buf* get(b200_buffer id) {
    auto it = bufs.find(id);
    if (it == bufs.end() || it->second.freed) return nullptr;
    return &it->second;
  }
  // A BFP8 buffer is read only by the ops that say so (`packed_ok`): every other op sees plain 16- or 32-bit
  // elements and is refused a packed one here, before it could misread the bytes.
  int need(b200_buffer id, Buf** out, const char* what, bool packed_ok = false) {
    Buf* b = get(id);
    if (!b) return fail(B200_STALE, "%s: buffer %llu is not live on this engine", what, (unsigned long long)id);
    if (b->elem == B200_BFP8 && !packed_ok)
      return fail(B200_UNSUPPORTED, "%s: buffer %llu is BFP8 storage; a product reads it as its B, cast_bfp widens it, nothing else reads it",
                  what, (unsigned long long)id);
    *out = b;
    return B200_OK;
  }
  void drop(b200_buffer id) {
    auto it = bufs.find(id);
    if (it == bufs.end()) return;
    Buf& b = it->second;
    if (b.views > 0) { b.freed = true; return; }
    const b200_buffer parent = b.parent;
    if (!b.parent && !b.adopted && b.ptr) release(b.ptr, b.bytes);
    bufs.erase(it);
    if (parent) {
      auto pit = bufs.find(parent);
      if (pit != bufs.end()) {
        pit->second.views--;
        if (pit->second.views == 0 && pit->second.freed) { pit->second.freed = false; drop(parent); }
      }
    }
  }
  // Host metadata (block lists, index lists) to a temporary device block.
  // Block lists (batched products, moves, attention heads) go to the device before their kernel.
  // A caller issues the same few lists every step, so lists of up to 64 KB are kept on the device
  // by content: a repeat costs no copy (and adds no copy node to a trace).  A kept list is owned by
  // the engine: *got comes back 0 and release() of it does nothing.
  struct MetaEntry { std::vector<uint8_t> bytes; void* dev = nullptr; };
  std::unordered_multimap<uint64_t, MetaEntry> meta_cache;
  uint64_t meta_hits = 0;
  static uint64_t fnv1a(const void* p, uint64_t n) {
    const uint8_t* b = (const uint8_t*)p;
    uint64_t h = 1469598103934665603ull;
    for (uint64_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
  }
  int to_device(const void* host, uint64_t bytes, void** dev, uint64_t* got) {
    const bool keepable = bytes > 0 && bytes <= (64u << 10);
    uint64_t key = 0;
    if (keepable) {
      key = fnv1a(host, bytes);
      auto range = meta_cache.equal_range(key);
      for (auto it = range.first; it != range.second; ++it)
        if (it->second.bytes.size() == bytes && memcmp(it->second.bytes.data(), host, bytes) == 0) {
          *dev = it->second.dev; *got = 0; ++meta_hits;
          return B200_OK;
        }
      if (!capturing && meta_cache.size() < 1024) {
        void* p = nullptr;
        if (cudaMalloc(&p, (bytes + 255) & ~255ull) == cudaSuccess) {
          auto it = meta_cache.emplace(key, MetaEntry());
          it->second.bytes.assign((const uint8_t*)host, (const uint8_t*)host + bytes);
          it->second.dev = p;
          cudaError_t e = cudaMemcpyAsync(p, it->second.bytes.data(), bytes, cudaMemcpyHostToDevice, stream);
          if (e != cudaSuccess) { cudaFree(p); meta_cache.erase(it); return cuda_fail(e, "metadata upload"); }
          traffic.bytes_h2d += bytes;
          *dev = p; *got = 0;
          return B200_OK;
        }
        cudaGetLastError();   // no room for a kept copy: the plain path below
      }
    }
    int st = alloc(bytes, dev, got);
    if (st) return st;
    if (capturing) {
      void* pin = nullptr;
      if (cudaMallocHost(&pin, bytes) != cudaSuccess) { cudaGetLastError(); release(*dev, *got); return fail(B200_OUT_OF_MEMORY, "trace: no pinned memory for a block list"); }
      memcpy(pin, host, bytes);
      cur.pinned.push_back(pin);
      host = pin;
    }
    cudaError_t e = cudaMemcpyAsync(*dev, host, bytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) { release(*dev, *got); return cuda_fail(e, "metadata upload"); }
    traffic.bytes_h2d += bytes;
    return B200_OK;
  }
  int launched(cudaError_t e, const char* what, int n = 1) {
    if (e == cudaErrorNotSupported) return fail(B200_UNSUPPORTED, "%s: unsupported", what);
    if (e != cudaSuccess) return cuda_fail(e, what);
    traffic.launches += n;
    if (capturing) { cur.launches += n; cur.ops.emplace_back(label, (uint64_t)n); }
    return B200_OK;
  }
  int wait() {
    if (capturing) return fail(B200_UNSUPPORTED, "a wait (download or sync) inside a trace capture");
    cudaError_t e = cudaMemcpyAsync(h_err, d_err, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) {
      sticky = B200_DEVICE;
      sticky_text = std::string("device failure: ") + cudaGetErrorString(e);
    } else if (*h_err != 0 && !sticky) {
      sticky = *h_err;
      sticky_text = sticky == B200_DOMAIN ? "DOMAIN: an index outside its table or a division by zero in an earlier op"
                                          : (sticky == B200_TIMEOUT ? "TIMEOUT: a bounded device wait ran out in an earlier op"
                                                                    : "an earlier op failed on the device");
    }
    if (sticky) { last_error = sticky_text; return sticky; }
    return B200_OK;
  }
};

namespace {

bool host_is_pinned(const void* p) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return at.type == cudaMemoryTypeHost;
}

int upload_any(b200_engine* e, const void* src, uint64_t rows, uint64_t cols, int elem, b200_buffer* out) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "upload inside a trace capture: upload before begin_trace and refresh with write");
  Buf* b = nullptr;
  int st = e->new_buffer(rows, cols, elem, out, &b);
  if (st) return st;
  const uint64_t bytes = rows * cols * elem_bytes(elem);
  if (bytes) {
    cudaError_t ce = cudaMemcpyAsync(b->ptr, src, bytes, cudaMemcpyHostToDevice, e->stream);
    if (ce != cudaSuccess) { e->drop(*out); return e->cuda_fail(ce, "upload"); }
    // A pinned source is read by DMA after the call returns; the trait lends the slice
    // only for the call, so wait for the copy.
    if (host_is_pinned(src)) cudaStreamSynchronize(e->stream);
  }
  e->traffic.bytes_h2d += bytes;
  e->traffic.h2d_calls++;
  return B200_OK;
}

int download_any(b200_engine* e, b200_buffer id, void* dst, uint64_t cap, int want_bytes, const char* what) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "%s inside a trace capture", what);
  Buf* b = nullptr;
  int st = e->need(id, &b, what);
  if (st) return st;
  if ((int)elem_bytes(b->elem) != want_bytes)
    return e->fail(B200_UNSUPPORTED, "%s: buffer %llu holds %d-byte elements", what, (unsigned long long)id, (int)elem_bytes(b->elem));
  const uint64_t n = b->rows * b->cols;
  if (cap < n) return e->fail(B200_UNSUPPORTED, "%s: %llu elements into room for %llu", what, (unsigned long long)n, (unsigned long long)cap);
  if (n) {
    cudaError_t ce = cudaMemcpyAsync(dst, b->ptr, n * want_bytes, cudaMemcpyDeviceToHost, e->stream);
    if (ce != cudaSuccess) return e->cuda_fail(ce, what);
  }
  e->traffic.bytes_d2h += n * want_bytes;
  e->traffic.d2h_calls++;
  return e->wait();
}

inline void set_dims(uint64_t d[2], uint64_t r, uint64_t c) { if (d) { d[0] = r; d[1] = c; } }

Mat mat_of(const Buf* b) {
  Mat m;
  m.p = b->ptr; m.ld = b->cols; m.rows = b->rows; m.cols = b->cols; m.bf16 = b->elem == B200_BF16;
  return m;
}
// A block of a buffer.
int mat_of_block(b200_engine* e, const b200_block_arg* a, Mat* m, const char* what) {
  Buf* b = nullptr;
  int st = e->need(a->id, &b, what);
  if (st) return st;
  if (a->at[0] + a->dims[0] > b->rows || a->at[1] + a->dims[1] > b->cols)
    return e->fail(B200_UNSUPPORTED, "%s: block [%llu,%llu]+[%llu,%llu] outside [%llu,%llu]", what,
                   (unsigned long long)a->at[0], (unsigned long long)a->at[1], (unsigned long long)a->dims[0],
                   (unsigned long long)a->dims[1], (unsigned long long)b->rows, (unsigned long long)b->cols);
  m->bf16 = b->elem == B200_BF16;
  m->p = (const char*)b->ptr + (a->at[0] * b->cols + a->at[1]) * elem_bytes(b->elem);
  m->ld = b->cols; m->rows = a->dims[0]; m->cols = a->dims[1];
  return B200_OK;
}

// How b meets a: the same shape, one row, one column, or whole rows repeated
// (crates/tt-kernels/src/tensor.rs:3799-3859).
bool broadcast_ok(uint32_t k, uint64_t rows, uint64_t cols, const Mat& b) {
  if (b.rows == rows && b.cols == cols) return true;
  if (!kind::broadcasts(k)) return false;
  if (b.rows == 1 && b.cols == cols) return true;
  if (b.cols == 1 && b.rows == rows) return true;
  if (b.cols == 1 && b.rows == 1) return true;
  if (b.cols == cols && b.rows > 0 && rows % b.rows == 0) return true;
  return false;
}

int run_eltwise(b200_engine* e, const b200_eltwise_op* op, Mat a, const Mat* b, const Mat* c, int out_bf16,
                b200_buffer* out, uint64_t out_dims[2]) {
  const uint32_t k = op->kind;
  const int ar = kind::arity(k);
  if (ar == 0) return e->fail(B200_UNSUPPORTED, "eltwise: kind %#x is not an element-wise op of this engine", k);
  if ((ar >= 2) != (b != nullptr) || (ar == 3) != (c != nullptr))
    return e->fail(B200_UNSUPPORTED, "eltwise %s: takes %d operand(s)", kind::name(k), ar);
  Mat bb, cc;
  if (b) bb = *b;
  if (c) cc = *c;
  // ADD and MUL take the broadcast operand on either side (crates/burn-tt/src/ops.rs:1850).
  if (b && (k == kind::ADD || k == kind::MUL) && (a.rows < bb.rows || a.cols < bb.cols)) std::swap(a, bb);
  const uint64_t rows = a.rows, cols = a.cols;
  if (b && !broadcast_ok(k, rows, cols, bb))
    return e->fail(B200_UNSUPPORTED, "eltwise %s: [%llu,%llu] with [%llu,%llu]", kind::name(k),
                   (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)bb.rows, (unsigned long long)bb.cols);
  if (c && (cc.rows != rows || cc.cols != cols))
    return e->fail(B200_UNSUPPORTED, "eltwise %s: third operand [%llu,%llu] is not [%llu,%llu]", kind::name(k),
                   (unsigned long long)cc.rows, (unsigned long long)cc.cols, (unsigned long long)rows, (unsigned long long)cols);
  if (k == kind::CLAMP && !(op->scalar <= op->scalar2))
    return e->fail(B200_UNSUPPORTED, "eltwise CLAMP: bounds %g, %g are crossed or NaN", op->scalar, op->scalar2);
  const int relem = kind::result_elem(k);
  if (out_bf16 && relem != 0) return e->fail(B200_UNSUPPORTED, "eltwise %s: a BF16 result of a non-float kind", kind::name(k));
  const int oelem = relem == 0 ? (out_bf16 ? B200_BF16 : B200_F32) : (relem == 1 ? B200_I32 : B200_BOOL);
  Buf* ob = nullptr;
  int st = e->new_buffer(rows, cols, oelem, out, &ob);
  if (st) return st;
  EltwiseArgs g{};
  g.kind = k; g.s1 = op->scalar; g.s2 = op->scalar2;
  g.a = a; g.b = bb; g.c = cc;
  g.out = ob->ptr; g.out_ld = cols; g.out_bf16 = out_bf16; g.rows = rows; g.cols = cols; g.err = e->d_err;
  st = e->launched(launch_eltwise(g, e->stream), "eltwise");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int copy_of(b200_engine* e, const Buf* src, b200_buffer* out, Buf** ob) {
  int st = e->new_buffer(src->rows, src->cols, src->elem, out, ob);
  if (st) return st;
  const uint64_t bytes = src->rows * src->cols * elem_bytes(src->elem);
  if (bytes) {
    cudaError_t ce = cudaMemcpyAsync((*ob)->ptr, src->ptr, bytes, cudaMemcpyDeviceToDevice, e->stream);
    if (ce != cudaSuccess) { e->drop(*out); return e->cuda_fail(ce, "copy"); }
  }
  return B200_OK;
}

int index_buf(b200_engine* e, b200_buffer id, Buf** b, const char* what) {
  int st = e->need(id, b, what);
  if (st) return st;
  if ((*b)->elem != B200_I32) return e->fail(B200_UNSUPPORTED, "%s: indices must be I32", what);
  return B200_OK;
}

}  // namespace

namespace b200 {
void set_global_error(const char* text) { set_create_error(text ? text : ""); }

namespace {
std::mutex g_device_lock;
std::map<std::pair<int, const void*>, size_t> g_smem_set;     // (device, kernel) -> bytes opted in
std::map<std::pair<int, const void*>, int> g_device_values;
}  // namespace

cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> hold(g_device_lock);
  size_t& have = g_smem_set[{dev, kernel}];
  if (have >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) have = bytes;
  return e;
}
bool device_value_get(const void* key, int* value) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> hold(g_device_lock);
  auto it = g_device_values.find({dev, key});
  if (it == g_device_values.end()) return false;
  *value = it->second;
  return true;
}
void device_value_set(const void* key, int value) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> hold(g_device_lock);
  g_device_values[{dev, key}] = value;
}
}  // namespace b200

extern "C" {

int32_t b200_engine_create(int32_t device_ordinal, const b200_config* cfg, b200_engine** out) {
  *out = nullptr;
  int count = 0;
  cudaError_t ce = cudaGetDeviceCount(&count);
  if (ce != cudaSuccess || count == 0) {
    cudaGetLastError();
    set_create_error(std::string("no CUDA device: ") + (ce != cudaSuccess ? cudaGetErrorString(ce) : "device count is 0"));
    return B200_NO_DEVICE;
  }
  if (device_ordinal < 0 || device_ordinal >= count) {
    set_create_error("no such device " + std::to_string(device_ordinal) + " (present: 0.." + std::to_string(count - 1) + ")");
    return B200_NO_DEVICE;
  }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, device_ordinal);
  if (prop.major != 10) {
    set_create_error(std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major) + std::to_string(prop.minor) +
                     "; this engine's kernels are built for sm_100a only");
    return B200_UNSUPPORTED;
  }
  if (cfg && (cfg->f32_matmul_mode < 0 || cfg->f32_matmul_mode > 2 || cfg->bf16_matmul_mode < 0 || cfg->bf16_matmul_mode > 2)) {
    set_create_error("config: unknown matmul mode");
    return B200_UNSUPPORTED;
  }
  b200_engine* e = new b200_engine();
  e->device = device_ordinal;
  if (cfg) e->cfg = *cfg;
  cudaSetDevice(device_ordinal);
  ce = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking);
  if (ce == cudaSuccess) ce = cudaEventCreate(&e->t0);
  if (ce == cudaSuccess) ce = cudaEventCreate(&e->t1);
  if (ce == cudaSuccess) ce = cudaMalloc(&e->d_err, 256);
  if (ce == cudaSuccess) ce = cudaMemsetAsync(e->d_err, 0, 256, e->stream);
  // words 2..3 of the error block: the limit of every bounded device wait, in clock cycles (0: the kernels' default)
  e->wait_limit_word = cfg ? (long long)cfg->wait_limit_cycles : 0;
  if (ce == cudaSuccess && e->wait_limit_word > 0)
    ce = cudaMemcpyAsync((char*)e->d_err + 8, &e->wait_limit_word, sizeof(long long), cudaMemcpyHostToDevice, e->stream);
  if (ce == cudaSuccess) ce = cudaMallocHost(&e->h_err, sizeof(int));
  if (ce == cudaSuccess) ce = cudaMalloc(&e->full_scratch, full_sum_scratch_floats() * sizeof(float));
  if (ce == cudaSuccess) ce = cudaMemsetAsync(e->full_scratch, 0, full_sum_scratch_floats() * sizeof(float), e->stream);
  if (ce != cudaSuccess) {
    set_create_error(std::string("engine set-up: ") + cudaGetErrorString(ce));
    delete e;
    return B200_DEVICE;
  }
  *e->h_err = 0;
  *out = e;
  return B200_OK;
}

void b200_engine_destroy(b200_engine* e) {
  if (!e) return;
  cudaSetDevice(e->device);
  cudaStreamSynchronize(e->stream);
  if (e->capturing) { cudaGraph_t g = nullptr; cudaStreamEndCapture(e->stream, &g); if (g) cudaGraphDestroy(g); cudaGetLastError(); }
  for (auto& kv : e->traces) {
    if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    if (kv.second.graph) cudaGraphDestroy(kv.second.graph);
    for (void* h : kv.second.pinned) cudaFreeHost(h);
    for (auto& b : kv.second.blocks) e->cache.emplace(b.second, b.first);  // freed with the cache below
  }
  for (auto it = e->bufs.begin(); it != e->bufs.end();) {  // buffers living in trace blocks are freed with them
    bool owned = false;
    for (auto& kv : e->traces) for (auto& b : kv.second.blocks) if (b.first == it->second.ptr) owned = true;
    it = owned ? e->bufs.erase(it) : std::next(it);
  }
  e->traces.clear();
  for (auto& kv : e->bufs)
    if (!kv.second.parent && !kv.second.adopted && kv.second.ptr) cudaFree(kv.second.ptr);
  for (auto& kv : e->cache) cudaFree(kv.second);
  for (auto& kv : e->meta_cache) cudaFree(kv.second.dev);
  e->drop_marks();
  cudaFree(e->d_err);
  cudaFree(e->full_scratch);
  cudaFreeHost(e->h_err);
  cudaEventDestroy(e->t0);
  cudaEventDestroy(e->t1);
  if (e->h2d_stream) cudaStreamDestroy(e->h2d_stream);
  if (e->d2h_stream) cudaStreamDestroy(e->d2h_stream);
  cudaStreamDestroy(e->stream);
  delete e;
}

int32_t b200_supports_dram(const b200_engine*) { return 1; }
int32_t b200_supports_batched_layout(const b200_engine*) { return 1; }
int32_t b200_supports_exact_matmul(const b200_engine*) { return 0; }

size_t b200_last_error(const b200_engine* e, char* buf, size_t len) {
  std::string global;
  if (!e) { std::lock_guard<std::mutex> hold(g_global_lock); global = g_create_error; }
  const std::string& s = e ? e->last_error : global;
  if (buf && len) {
    const size_t n = std::min(len - 1, s.size());
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return s.size();
}
void b200_last_oom(const b200_engine* e, uint64_t out[3]) { out[0] = e->oom[0]; out[1] = e->oom[1]; out[2] = e->oom[2]; }

// ---- storage -------------------------------------------------------------------
int32_t b200_upload_f32(b200_engine* e, const float* v, uint64_t rows, uint64_t cols, b200_buffer* out) {
  return upload_any(e, v, rows, cols, B200_F32, out);
}
int32_t b200_upload_bf16(b200_engine* e, const uint16_t* v, uint64_t rows, uint64_t cols, b200_buffer* out) {
  return upload_any(e, v, rows, cols, B200_BF16, out);
}
int32_t b200_upload_bits(b200_engine* e, const uint32_t* v, uint64_t rows, uint64_t cols, int32_t elem, b200_buffer* out) {
  if (elem != B200_F32 && elem != B200_I32 && elem != B200_BOOL)
    return e->fail(B200_UNSUPPORTED, "upload_bits: elem %d is not a 32-bit element", elem);
  return upload_any(e, v, rows, cols, elem, out);
}
int32_t b200_download_f32(b200_engine* e, b200_buffer id, float* out, uint64_t cap) {
  Buf* b = e->get(id);
  if (b && b->elem != B200_F32) return e->fail(B200_UNSUPPORTED, "download: buffer %llu is not F32", (unsigned long long)id);
  return download_any(e, id, out, cap, 4, "download");
}
int32_t b200_download_bf16(b200_engine* e, b200_buffer id, uint16_t* out, uint64_t cap) {
  return download_any(e, id, out, cap, 2, "download_bf16");
}
int32_t b200_download_bits(b200_engine* e, b200_buffer id, uint32_t* out, uint64_t cap) {
  return download_any(e, id, out, cap, 4, "download_bits");
}
void b200_free(b200_engine* e, b200_buffer id) { e->drop(id); }

int32_t b200_zeros(b200_engine* e, uint64_t rows, uint64_t cols, int32_t elem, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  if (elem < 0 || elem > B200_BF16) return e->fail(B200_UNSUPPORTED, "zeros: unknown elem %d", elem);
  Buf* b = nullptr;
  int st = e->new_buffer(rows, cols, elem, out, &b);
  if (st) return st;
  const uint64_t bytes = rows * cols * elem_bytes(elem);
  if (bytes) {
    cudaError_t ce = cudaMemsetAsync(b->ptr, 0, bytes, e->stream);
    if (ce != cudaSuccess) { e->drop(*out); return e->cuda_fail(ce, "zeros"); }
  }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_dims(const b200_engine* e, b200_buffer id, uint64_t out_dims[2], int32_t* elem) {
  auto it = e->bufs.find(id);
  if (it == e->bufs.end() || it->second.freed) return B200_STALE;
  set_dims(out_dims, it->second.rows, it->second.cols);
  if (elem) *elem = it->second.elem;
  return B200_OK;
}
int32_t b200_device_ptr(const b200_engine* e, b200_buffer id, void** ptr, uint64_t* bytes) {
  auto it = e->bufs.find(id);
  if (it == e->bufs.end() || it->second.freed) return B200_STALE;
  *ptr = it->second.ptr;
  if (bytes) *bytes = it->second.rows * it->second.cols * elem_bytes(it->second.elem);
  return B200_OK;
}
int32_t b200_adopt(b200_engine* e, void* p, uint64_t rows, uint64_t cols, int32_t elem, b200_buffer* out) {
  if (elem < 0 || elem > B200_BF16) return e->fail(B200_UNSUPPORTED, "adopt: unknown elem %d", elem);
  if (reinterpret_cast<uintptr_t>(p) & 15) return e->fail(B200_UNSUPPORTED, "adopt: address is not 16-byte aligned");
  Buf b;
  b.ptr = p; b.rows = rows; b.cols = cols; b.elem = elem; b.adopted = true;
  *out = e->next_id++;
  e->bufs.emplace(*out, b);
  return B200_OK;
}
int32_t b200_copy_into(b200_engine* e, b200_buffer src, b200_buffer dst) {
  cudaSetDevice(e->device);
  Buf *s = nullptr, *d = nullptr;
  int st = e->need(src, &s, "copy_into");
  if (!st) st = e->need(dst, &d, "copy_into");
  if (st) return st;
  if (s->rows != d->rows || s->cols != d->cols || s->elem != d->elem)
    return e->fail(B200_UNSUPPORTED, "copy_into: [%llu,%llu] into [%llu,%llu]", (unsigned long long)s->rows,
                   (unsigned long long)s->cols, (unsigned long long)d->rows, (unsigned long long)d->cols);
  cudaError_t ce = cudaMemcpyAsync(d->ptr, s->ptr, s->rows * s->cols * elem_bytes(s->elem), cudaMemcpyDeviceToDevice, e->stream);
  return ce == cudaSuccess ? B200_OK : e->cuda_fail(ce, "copy_into");
}
static int write_any(b200_engine* e, b200_buffer id, const void* v, uint64_t n, int eb) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "write inside a trace capture");
  Buf* b = nullptr;
  int st = e->need(id, &b, "write");
  if (st) return st;
  if (b->rows * b->cols != n || (int)elem_bytes(b->elem) != eb)
    return e->fail(B200_UNSUPPORTED, "write: %llu elements of %d bytes into [%llu,%llu]", (unsigned long long)n, eb,
                   (unsigned long long)b->rows, (unsigned long long)b->cols);
  cudaError_t ce = cudaMemcpyAsync(b->ptr, v, n * eb, cudaMemcpyHostToDevice, e->stream);
  if (ce != cudaSuccess) return e->cuda_fail(ce, "write");
  e->traffic.bytes_h2d += n * eb;
  e->traffic.h2d_calls++;
  return B200_OK;
}
int32_t b200_write_f32(b200_engine* e, b200_buffer id, const float* v, uint64_t n) { return write_any(e, id, v, n, 4); }
int32_t b200_write_bf16(b200_engine* e, b200_buffer id, const uint16_t* v, uint64_t n) { return write_any(e, id, v, n, 2); }

// ---- products -------------------------------------------------------------------
static int run_gemm(b200_engine* e, GemmArgs& g, const GemmBatch* batches_host, const char* what) {
  const char* why = "";
  g.sm_limit = e->matmul_sm_limit;
  const bool want_tc = g.in_bf16 ? e->cfg.bf16_matmul_mode != 1 : e->cfg.f32_matmul_mode == 2;
  // A handful of rows (a decode step): stream B once instead of a 128-row tile with a few live rows.
  if (g.in_bf16 && e->cfg.bf16_matmul_mode == 0 && gemm_skinny_supported(g)) {
    e->matmul_path = "skinny";
    return e->launched(launch_gemm_skinny(g, e->stream), what);
  }
  if (want_tc && gemm_tc_supported(g, &why)) {
    int pair = 0;
    const cudaError_t ce = launch_gemm_tc(g, batches_host, e->d_err, e->stream, &pair);
    if (ce != cudaErrorNotSupported) {
      e->matmul_path = pair ? "tcgen05-pair" : "tcgen05";
      return e->launched(ce, what);
    }
    why = "the driver refused a tensor map for this shape";
  }
  if (g.in_bf16 && e->cfg.bf16_matmul_mode == 2)
    return e->fail(B200_UNSUPPORTED, "%s: the tcgen05 path refuses this product (%s) and the engine is set to use no other", what, why);
  // F32 operands: the split-TF32 tensor-core kernel for products large enough to pay for the
  // split (automatic from 256^3 up), else FMA.  f32_matmul_mode 1 = FMA only, 2 = tensor only.
  if (!g.in_bf16 && e->cfg.f32_matmul_mode != 1) {
    const bool big = g.m >= 256 && g.n >= 256 && g.k >= 256;
    if ((big || e->cfg.f32_matmul_mode == 2) && gemm_tf32_supported(g, &why)) {
      const uint64_t a_rows = g.a_trans ? g.k : g.m, b_rows = g.b_trans ? g.n : g.k;
      const uint64_t na = a_rows * g.lda * 4, nb = b_rows * g.ldb * 4;
      void* t[4] = {nullptr, nullptr, nullptr, nullptr};
      uint64_t got[4] = {0, 0, 0, 0};
      int st = B200_OK;
      for (int i = 0; i < 4 && !st; ++i) st = e->alloc(i < 2 ? na : nb, &t[i], &got[i]);
      cudaError_t ce = cudaErrorMemoryAllocation;
      if (!st) ce = launch_gemm_tf32(g, t[0], t[1], t[2], t[3], e->d_err, e->stream);
      for (int i = 0; i < 4; ++i) if (t[i]) e->release(t[i], got[i]);
      if (st) return st;
      if (ce != cudaErrorNotSupported) {
        e->matmul_path = "tcgen05-tf32x3";
        return e->launched(ce, what, 3);
      }
      why = "the driver refused a tensor map for this shape";
    }
    if (e->cfg.f32_matmul_mode == 2)
      return e->fail(B200_UNSUPPORTED, "%s: the split-TF32 path refuses this product (%s) and the engine is set to use no other", what, why);
  }
  e->matmul_path = "simt";
  return e->launched(launch_gemm_simt(g, e->stream), what);
}

int32_t b200_matmul(b200_engine* e, b200_buffer a, int32_t ta, b200_buffer b, int32_t tb, int32_t out_bf16,
                    b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr;
  int st = e->need(a, &A, "matmul");
  if (!st) st = e->need(b, &B, "matmul", true);
  if (st) return st;
  if (B->elem == B200_BFP8) {
    // A weight kept as BFP8 (crates/burn-tt/src/storage.rs:117-123): a BF16 activation of a few rows reads it where it
    // lies, decoding in the product's load path; anything else multiplies by the weight widened for the call --
    // bit for bit the product with the decoded values either way (every decoded value is a BF16 value).
    if (A->elem != B200_BF16 && A->elem != B200_F32) return e->fail(B200_UNSUPPORTED, "matmul: A must be F32 or BF16 against a BFP8 B");
    const uint64_t m = ta ? A->cols : A->rows, k = ta ? A->rows : A->cols;
    if (!ta && !tb && A->elem == B200_BF16 && B->rows == k && k > 0 && gemm_skinny_bfp_supported(m, B->cols, k) &&
        e->cfg.bf16_matmul_mode == 0) {
      const uint64_t n = B->cols;
      Buf* C = nullptr;
      st = e->new_buffer(m, n, out_bf16 ? B200_BF16 : B200_F32, out, &C);
      if (st) return st;
      A = e->get(a); B = e->get(b);
      const uint8_t* datums = (const uint8_t*)B->ptr;
      st = e->launched(launch_gemm_skinny_bfp((const uint16_t*)A->ptr, A->cols, datums, datums + B->rows * B->cols, C->ptr, n, out_bf16,
                                              m, n, k, e->stream), "matmul");
      if (st) { e->drop(*out); return st; }
      e->matmul_path = "skinny-bfp8";
      set_dims(out_dims, m, n);
      return B200_OK;
    }
    b200_buffer wide = 0; uint64_t wd[2];
    st = b200_cast_bfp(e, b, A->elem == B200_BF16 ? -16 : 0, &wide, wd);
    if (st) return st;
    st = b200_matmul(e, a, ta, wide, tb, out_bf16, out, out_dims);
    e->drop(wide);
    return st;
  }
  const bool abf = A->elem == B200_BF16, bbf = B->elem == B200_BF16;
  if ((A->elem != B200_F32 && !abf) || (B->elem != B200_F32 && !bbf))
    return e->fail(B200_UNSUPPORTED, "matmul: operands must be F32 or BF16 (got elem %d, %d)", A->elem, B->elem);
  if (abf != bbf) {
    // An F32 operand against one kept in BF16 storage (`cast_bf16_storage`, crates/burn-tt/src/server.rs:150;
    // crates/tt-kernels/src/session.rs:3751-3756): bit for bit the F32 product with the stored operand widened,
    // so it is widened into a block that lives for this product and the F32 path runs.
    b200_buffer wide = 0; uint64_t wd[2];
    st = b200_cast_float(e, abf ? a : b, 0, &wide, wd);
    if (st) return st;
    st = b200_matmul(e, abf ? wide : a, ta, abf ? b : wide, tb, out_bf16, out, out_dims);
    e->drop(wide);
    return st;
  }
  const uint64_t m = ta ? A->cols : A->rows, k = ta ? A->rows : A->cols;
  const uint64_t k2 = tb ? B->cols : B->rows, n = tb ? B->rows : B->cols;
  if (k != k2)
    return e->fail(B200_UNSUPPORTED, "matmul: [%llu,%llu] x [%llu,%llu]", (unsigned long long)m, (unsigned long long)k,
                   (unsigned long long)k2, (unsigned long long)n);
  Buf* C = nullptr;
  st = e->new_buffer(m, n, out_bf16 ? B200_BF16 : B200_F32, out, &C);
  if (st) return st;
  // new_buffer may rehash the table
  A = e->get(a); B = e->get(b);
  GemmArgs g{};
  g.a = A->ptr; g.b = B->ptr; g.c = C->ptr;
  g.in_bf16 = abf; g.out_bf16 = out_bf16;
  g.m = m; g.n = n; g.k = k;
  g.lda = A->cols; g.ldb = B->cols; g.ldc = n;
  g.a_trans = ta; g.b_trans = tb;
  g.batch = 1; g.batches_dev = nullptr;
  if (k == 0) {
    cudaMemsetAsync(C->ptr, 0, m * n * elem_bytes(C->elem), e->stream);
  } else {
    st = run_gemm(e, g, nullptr, "matmul");
    if (st) { e->drop(*out); return st; }
  }
  set_dims(out_dims, m, n);
  return B200_OK;
}

int32_t b200_matmul_host(b200_engine* e, const float* a, const float* b, const uint64_t mkn[3], float* out) {
  b200_buffer ia = 0, ib = 0, ic = 0;
  uint64_t d[2];
  int st = b200_upload_f32(e, a, mkn[0], mkn[1], &ia);
  if (!st) st = b200_upload_f32(e, b, mkn[1], mkn[2], &ib);
  if (!st) st = b200_matmul(e, ia, 0, ib, 0, 0, &ic, d);
  if (!st) st = b200_download_f32(e, ic, out, mkn[0] * mkn[2]);
  b200_free(e, ia); b200_free(e, ib); b200_free(e, ic);
  return st;
}

// silu(A Bg) * (A Bu) as one product: B holds the gate and up weights interleaved in groups of 128
// columns (columns [256t, 256t+128) are gate columns 128t.., the next 128 the matching up columns),
// so a 256-wide tile of the product holds both and its epilogue stores the activation.  Bit for bit
// `matmul_dram_bf16` on [Bg | Bu] followed by `SILU_MUL` on its halves (tt-models/src/llama.rs:498).
int32_t b200_matmul_silu_mul(b200_engine* e, b200_buffer a, b200_buffer b, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr;
  int st = e->need(a, &A, "matmul_silu_mul");
  if (!st) st = e->need(b, &B, "matmul_silu_mul");
  if (st) return st;
  if (A->elem != B200_BF16 || B->elem != B200_BF16) return e->fail(B200_UNSUPPORTED, "matmul_silu_mul: BF16 operands");
  const uint64_t m = A->rows, k = A->cols, n = B->cols;
  if (B->rows != k || k == 0 || m == 0 || n == 0 || n % 256)
    return e->fail(B200_UNSUPPORTED, "matmul_silu_mul: [%llu,%llu] x [%llu,%llu] (the weights come in groups of 256 columns)",
                   (unsigned long long)m, (unsigned long long)k, (unsigned long long)B->rows, (unsigned long long)n);
  Buf* C = nullptr;
  st = e->new_buffer(m, n / 2, B200_BF16, out, &C);
  if (st) return st;
  A = e->get(a); B = e->get(b);
  GemmArgs g{};
  g.a = A->ptr; g.b = B->ptr; g.c = C->ptr;
  g.in_bf16 = 1; g.out_bf16 = 1;
  g.m = m; g.n = n; g.k = k;
  g.lda = A->cols; g.ldb = B->cols; g.ldc = n / 2;
  g.a_trans = 0; g.b_trans = 0; g.batch = 1; g.batches_dev = nullptr;
  g.epi_mode = 1;
  g.sm_limit = e->matmul_sm_limit;
  const char* why = "";
  if (!gemm_tc_supported(g, &why)) { e->drop(*out); return e->fail(B200_UNSUPPORTED, "matmul_silu_mul: the tcgen05 path refuses this product (%s)", why); }
  int pair = 0;
  const cudaError_t ce = launch_gemm_tc(g, nullptr, e->d_err, e->stream, &pair);
  if (ce == cudaErrorNotSupported) { e->drop(*out); return e->fail(B200_UNSUPPORTED, "matmul_silu_mul: the driver refused a tensor map for this shape"); }
  e->matmul_path = pair ? "tcgen05-pair" : "tcgen05";
  st = e->launched(ce, "matmul_silu_mul");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, m, n / 2);
  return B200_OK;
}

// The fused QKV projection with RoPE applied in the product's epilogue to the heads below `rope_cols` (the query and
// key heads; the value heads pass through): bit for bit `matmul_dram_bf16` then `rope_blocks` with a BF16 result on
// those columns (crates/tt-models/src/llama.rs:404-433), without the second launch or its pass over the projection.
int32_t b200_matmul_rope(b200_engine* e, b200_buffer a, b200_buffer b, const b200_block_arg* cs, const b200_block_arg* sn,
                         uint64_t rope_cols, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr;
  int st = e->need(a, &A, "matmul_rope");
  if (!st) st = e->need(b, &B, "matmul_rope");
  if (st) return st;
  Mat mc, ms;
  st = mat_of_block(e, cs, &mc, "matmul_rope");
  if (!st) st = mat_of_block(e, sn, &ms, "matmul_rope");
  if (st) return st;
  A = e->get(a); B = e->get(b);
  if (A->elem != B200_BF16 || B->elem != B200_BF16) return e->fail(B200_UNSUPPORTED, "matmul_rope: BF16 operands");
  const uint64_t m = A->rows, k = A->cols, n = B->cols;
  if (B->rows != k || k == 0 || m == 0 || n == 0 || rope_cols == 0 || rope_cols % 64 || rope_cols > n)
    return e->fail(B200_UNSUPPORTED, "matmul_rope: [%llu,%llu] x [%llu,%llu] with RoPE on %llu columns (heads of 64 within the product)",
                   (unsigned long long)m, (unsigned long long)k, (unsigned long long)B->rows, (unsigned long long)n, (unsigned long long)rope_cols);
  auto table_ok = [&](const Mat& t) {
    return !t.bf16 && t.cols == 64 && t.rows > 0 && m % t.rows == 0 && t.ld % 4 == 0 && ((uintptr_t)t.p & 15) == 0 && t.ld < (1ull << 31) &&
           t.rows < (1ull << 31);
  };
  if (!table_ok(mc) || !table_ok(ms) || mc.rows != ms.rows || mc.ld != ms.ld)
    return e->fail(B200_UNSUPPORTED, "matmul_rope: the tables are F32 [r, 64] blocks at 16-byte rows, r dividing the product's rows");
  Buf* C = nullptr;
  st = e->new_buffer(m, n, B200_BF16, out, &C);
  if (st) return st;
  A = e->get(a); B = e->get(b);
  GemmArgs g{};
  g.a = A->ptr; g.b = B->ptr; g.c = C->ptr;
  g.in_bf16 = 1; g.out_bf16 = 1;
  g.m = m; g.n = n; g.k = k;
  g.lda = A->cols; g.ldb = B->cols; g.ldc = n;
  g.a_trans = 0; g.b_trans = 0; g.batch = 1; g.batches_dev = nullptr;
  g.epi_mode = 2;
  g.rope_cos = (const float*)mc.p; g.rope_sin = (const float*)ms.p;
  g.rope_rows = (uint32_t)mc.rows; g.rope_ld = (uint32_t)mc.ld; g.rope_cols = (uint32_t)rope_cols;
  g.sm_limit = e->matmul_sm_limit;
  const char* why = "";
  if (n >= (1ull << 31) || !gemm_tc_supported(g, &why)) { e->drop(*out); return e->fail(B200_UNSUPPORTED, "matmul_rope: the tcgen05 path refuses this product (%s)", why); }
  int pair = 0;
  const cudaError_t ce = launch_gemm_tc(g, nullptr, e->d_err, e->stream, &pair);
  if (ce == cudaErrorNotSupported) { e->drop(*out); return e->fail(B200_UNSUPPORTED, "matmul_rope: the driver refused a tensor map for this shape"); }
  e->matmul_path = pair ? "tcgen05-pair" : "tcgen05";
  st = e->launched(ce, "matmul_rope");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, m, n);
  return B200_OK;
}

int32_t b200_matmul_add_rms_norm(b200_engine* e, b200_buffer a, b200_buffer b, b200_buffer resid, b200_buffer gains, float eps,
                                 b200_buffer out[2], uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr, *R = nullptr, *G = nullptr;
  int st = e->need(a, &A, "matmul_add_rms_norm");
  if (!st) st = e->need(b, &B, "matmul_add_rms_norm");
  if (!st) st = e->need(resid, &R, "matmul_add_rms_norm");
  if (!st) st = e->need(gains, &G, "matmul_add_rms_norm");
  if (st) return st;
  if (A->elem != B200_BF16 || B->elem != B200_BF16 || R->elem != B200_F32 || G->elem != B200_BF16)
    return e->fail(B200_UNSUPPORTED, "matmul_add_rms_norm: BF16 operands and gains, an F32 residual");
  const uint64_t m = A->rows, k = A->cols, n = B->cols;
  if (B->rows != k || R->rows != m || R->cols != n || G->rows * G->cols != n)
    return e->fail(B200_UNSUPPORTED, "matmul_add_rms_norm: [%llu,%llu] x [%llu,%llu] + [%llu,%llu] with %llu gains: the shapes do not meet",
                   (unsigned long long)m, (unsigned long long)k, (unsigned long long)B->rows, (unsigned long long)n,
                   (unsigned long long)R->rows, (unsigned long long)R->cols, (unsigned long long)(G->rows * G->cols));
  const char* why = "";
  if (!gemm_addnorm_supported(m, n, k, &why)) return e->fail(B200_UNSUPPORTED, "matmul_add_rms_norm: %s", why);
  Buf *S = nullptr, *N = nullptr;
  st = e->new_buffer(m, n, B200_F32, &out[0], &S);
  if (st) return st;
  st = e->new_buffer(m, n, B200_BF16, &out[1], &N);
  if (st) { e->drop(out[0]); return st; }
  A = e->get(a); B = e->get(b); R = e->get(resid); G = e->get(gains); S = e->get(out[0]);
  const cudaError_t ce = launch_gemm_addnorm(A->ptr, B->ptr, (const float*)R->ptr, G->ptr, eps, (float*)S->ptr, N->ptr, m, n, k, e->d_err, e->stream);
  if (ce == cudaErrorNotSupported) {
    e->drop(out[0]); e->drop(out[1]);
    return e->fail(B200_UNSUPPORTED, "matmul_add_rms_norm: the driver refused a tensor map for this shape");
  }
  e->matmul_path = "tcgen05-addnorm";
  st = e->launched(ce, "matmul_add_rms_norm");
  if (st) { e->drop(out[0]); e->drop(out[1]); return st; }
  set_dims(out_dims, m, n);
  return B200_OK;
}

// C = A B written into one or more caller-named matrices instead of a new buffer: the sharded
// product's rank writes its column slice straight into every rank's C (its own and, through
// addresses opened with b200_ipc_open, its peers' over NVLink) from the product's epilogue.
static int matmul_into_any(b200_engine* e, b200_buffer a, b200_buffer b, void* const* dst, int32_t n_dst, uint64_t dst_rows,
                           uint64_t dst_cols, uint64_t col_first, int32_t out_bf16, int multicast) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr;
  int st = e->need(a, &A, "matmul_into");
  if (!st) st = e->need(b, &B, "matmul_into");
  if (st) return st;
  if (A->elem != B200_BF16 || B->elem != B200_BF16) return e->fail(B200_UNSUPPORTED, "matmul_into: BF16 operands");
  const uint64_t m = A->rows, k = A->cols, n = B->cols;
  if (B->rows != k) return e->fail(B200_UNSUPPORTED, "matmul_into: [%llu,%llu] x [%llu,%llu]", (unsigned long long)m, (unsigned long long)k,
                                   (unsigned long long)B->rows, (unsigned long long)n);
  if (n_dst < 1 || n_dst > 8 || !dst) return e->fail(B200_UNSUPPORTED, "matmul_into: 1 to 8 destinations");
  for (int i = 0; i < n_dst; ++i) if (!dst[i]) return e->fail(B200_UNSUPPORTED, "matmul_into: destination %d is null", i);
  if (m != dst_rows || col_first + n > dst_cols)
    return e->fail(B200_UNSUPPORTED, "matmul_into: a [%llu,%llu] product at column %llu of [%llu,%llu]", (unsigned long long)m,
                   (unsigned long long)n, (unsigned long long)col_first, (unsigned long long)dst_rows, (unsigned long long)dst_cols);
  if (k == 0 || m == 0 || n == 0) return e->fail(B200_UNSUPPORTED, "matmul_into: an empty product");
  const uint64_t eb = out_bf16 ? 2 : 4;
  // A multicast address takes whole 16-byte pieces of whole 128-byte row segments only (one multimem.st each): no ragged edge
  if (multicast && (n_dst != 1 || (n * eb) % 128 || (col_first * eb) % 16 || (dst_cols * eb) % 16 || ((uintptr_t)dst[0] & 15)))
    return e->fail(B200_UNSUPPORTED, "matmul_into_multicast: %llu columns at column %llu of %llu are not whole 128-byte row segments at 16-byte addresses",
                   (unsigned long long)n, (unsigned long long)col_first, (unsigned long long)dst_cols);
  GemmArgs g{};
  g.a = A->ptr; g.b = B->ptr;
  g.c = (char*)dst[0] + col_first * eb;
  g.n_more = n_dst - 1;
  for (int i = 1; i < n_dst; ++i) g.c_more[i - 1] = (char*)dst[i] + col_first * eb;
  g.in_bf16 = 1; g.out_bf16 = out_bf16;
  g.m = m; g.n = n; g.k = k;
  g.lda = A->cols; g.ldb = B->cols; g.ldc = dst_cols;
  g.a_trans = 0; g.b_trans = 0; g.batch = 1; g.batches_dev = nullptr;
  g.sm_limit = e->matmul_sm_limit;
  g.multicast = multicast;
  const char* why = "";
  if (!gemm_tc_supported(g, &why)) return e->fail(B200_UNSUPPORTED, "matmul_into: the tcgen05 path refuses this product (%s)", why);
  int pair = 0;
  const cudaError_t ce = launch_gemm_tc(g, nullptr, e->d_err, e->stream, &pair);
  if (ce == cudaErrorNotSupported) return e->fail(B200_UNSUPPORTED, "matmul_into: the driver refused a tensor map for this shape");
  e->matmul_path = pair ? "tcgen05-pair" : "tcgen05";
  return e->launched(ce, "matmul_into");
}
int32_t b200_matmul_into(b200_engine* e, b200_buffer a, b200_buffer b, void* const* dst, int32_t n_dst, uint64_t dst_rows,
                         uint64_t dst_cols, uint64_t col_first, int32_t out_bf16) {
  return matmul_into_any(e, a, b, dst, n_dst, dst_rows, dst_cols, col_first, out_bf16, 0);
}
// The same product stored ONCE, at a multicast address that maps every rank's C (an NVLS multicast object):
// the NVSwitch replicates each store to every GPU of the group, so a rank's outbound bytes are its slice, not
// its slice times the other ranks.
int32_t b200_matmul_into_multicast(b200_engine* e, b200_buffer a, b200_buffer b, void* multicast_dst, uint64_t dst_rows,
                                   uint64_t dst_cols, uint64_t col_first, int32_t out_bf16) {
  void* const one[1] = {multicast_dst};
  if (!multicast_dst) return e->fail(B200_UNSUPPORTED, "matmul_into_multicast: the destination is null");
  return matmul_into_any(e, a, b, one, 1, dst_rows, dst_cols, col_first, out_bf16, 1);
}

// A block of a buffer stored into columns [col_first, ...) of each of the n_dst matrices dst[i]
// ([dst_rows, dst_cols] of the block's type; this GPU's or a peer's): a rank's column slice of an
// all-gather, written everywhere by its owner.
static int store_block_any(b200_engine* e, const b200_block_arg* src, void* const* dst, int32_t n_dst, uint64_t dst_rows,
                           uint64_t dst_cols, uint64_t col_first, int multicast) {
  cudaSetDevice(e->device);
  Buf* S = nullptr;
  int st = e->need(src->id, &S, "store_block_into");
  if (st) return st;
  const uint64_t rows = src->dims[0], cols = src->dims[1];
  if (src->at[0] + rows > S->rows || src->at[1] + cols > S->cols || rows != dst_rows || col_first + cols > dst_cols)
    return e->fail(B200_UNSUPPORTED, "store_block_into: shapes do not meet");
  if (n_dst < 1 || n_dst > 8 || !dst) return e->fail(B200_UNSUPPORTED, "store_block_into: 1 to 8 destinations");
  for (int i = 0; i < n_dst; ++i) if (!dst[i]) return e->fail(B200_UNSUPPORTED, "store_block_into: destination %d is null", i);
  const uint64_t eb = elem_bytes(S->elem);
  const char* sp = (const char*)S->ptr + (src->at[0] * S->cols + src->at[1]) * eb;
  void* shifted[8];
  for (int i = 0; i < n_dst; ++i) shifted[i] = (char*)dst[i] + col_first * eb;
  const cudaError_t ce = launch_store_block_many(sp, S->cols * eb, shifted, n_dst, dst_cols * eb, rows, cols * eb, multicast, e->stream);
  if (ce == cudaErrorNotSupported) return e->fail(B200_UNSUPPORTED, "store_block_into: rows are not whole 16-byte pieces at 16-byte addresses");
  return e->launched(ce, "store_block_into");
}
int32_t b200_store_block_into(b200_engine* e, const b200_block_arg* src, void* const* dst, int32_t n_dst, uint64_t dst_rows,
                              uint64_t dst_cols, uint64_t col_first) {
  return store_block_any(e, src, dst, n_dst, dst_rows, dst_cols, col_first, 0);
}
int32_t b200_store_block_into_multicast(b200_engine* e, const b200_block_arg* src, void* multicast_dst, uint64_t dst_rows,
                                        uint64_t dst_cols, uint64_t col_first) {
  void* const one[1] = {multicast_dst};
  if (!multicast_dst) return e->fail(B200_UNSUPPORTED, "store_block_into_multicast: the destination is null");
  return store_block_any(e, src, one, 1, dst_rows, dst_cols, col_first, 1);
}

// Another process's view of a buffer of this engine (CUDA IPC): export here, open there.
int32_t b200_ipc_export(b200_engine* e, b200_buffer buf, uint8_t handle[64]) {
  cudaSetDevice(e->device);
  Buf* X = nullptr;
  int st = e->need(buf, &X, "ipc_export");
  if (st) return st;
  if (X->parent || X->adopted) return e->fail(B200_UNSUPPORTED, "ipc_export: a view or an adopted buffer has no allocation of its own");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the ABI carries a 64-byte handle");
  cudaIpcMemHandle_t h;
  const cudaError_t ce = cudaIpcGetMemHandle(&h, X->ptr);
  if (ce != cudaSuccess) return e->cuda_fail(ce, "ipc_export");
  memcpy(handle, &h, 64);
  return B200_OK;
}
int32_t b200_ipc_open(b200_engine* e, const uint8_t handle[64], void** ptr) {
  cudaSetDevice(e->device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  const cudaError_t ce = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (ce != cudaSuccess) { cudaGetLastError(); return e->cuda_fail(ce, "ipc_open"); }
  return B200_OK;
}
int32_t b200_ipc_close(b200_engine* e, void* ptr) {
  cudaSetDevice(e->device);
  const cudaError_t ce = cudaIpcCloseMemHandle(ptr);
  return ce == cudaSuccess ? B200_OK : e->cuda_fail(ce, "ipc_close");
}

// The host-staged product for BF16 operands, with its copies overlapped: B goes up whole, then A
// goes up, is multiplied and its rows of C come down in row panels, so the upload of panel p+1, the
// product of panel p and the download of panel p-1 run at once (PCIe carries both directions).  Returns
// when C is complete in `out`.  Pinned host memory gives the overlap; pageable memory still works.
int32_t b200_matmul_host_bf16(b200_engine* e, const uint16_t* a, const uint16_t* b, const uint64_t mkn[3], uint16_t* out) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "matmul_host_bf16 inside a trace capture");
  const uint64_t m = mkn[0], k = mkn[1], n = mkn[2];
  if (m == 0 || n == 0) return B200_OK;
  if (k == 0) { memset(out, 0, m * n * 2); return B200_OK; }
  if (!e->h2d_stream) {
    cudaError_t ce = cudaStreamCreateWithFlags(&e->h2d_stream, cudaStreamNonBlocking);
    if (ce == cudaSuccess) ce = cudaStreamCreateWithFlags(&e->d2h_stream, cudaStreamNonBlocking);
    if (ce != cudaSuccess) return e->cuda_fail(ce, "matmul_host_bf16: streams");
  }
  // panels of about 1024 rows (whole 256-row tiles), at most 64 of them
  uint64_t rows = 1024;
  while ((m + rows - 1) / rows > 64) rows *= 2;
  if (rows > m) rows = m;
  const uint64_t panels = (m + rows - 1) / rows;
  void *da = nullptr, *db = nullptr, *dc = nullptr;
  uint64_t ga = 0, gb = 0, gc = 0;
  int st = e->alloc(m * k * 2, &da, &ga);
  if (!st) st = e->alloc(k * n * 2, &db, &gb);
  if (!st) st = e->alloc(m * n * 2, &dc, &gc);
  std::vector<cudaEvent_t> ev(2 * panels + 2, nullptr);
  cudaError_t ce = cudaSuccess;
  for (auto& x : ev) if (!st && ce == cudaSuccess) ce = cudaEventCreateWithFlags(&x, cudaEventDisableTiming);
  if (!st && ce != cudaSuccess) st = e->cuda_fail(ce, "matmul_host_bf16: events");
  if (!st) {
    cudaEvent_t start = ev[2 * panels], b_up = ev[2 * panels + 1];
    // the pool's blocks may still be read by work already on the engine's stream
    cudaEventRecord(start, e->stream);
    cudaStreamWaitEvent(e->h2d_stream, start, 0);
    ce = cudaMemcpyAsync(db, b, k * n * 2, cudaMemcpyHostToDevice, e->h2d_stream);
    cudaEventRecord(b_up, e->h2d_stream);
    cudaStreamWaitEvent(e->stream, b_up, 0);
    for (uint64_t p = 0; p < panels && ce == cudaSuccess && !st; ++p) {
      const uint64_t r0 = p * rows, nr = (r0 + rows <= m) ? rows : m - r0;
      ce = cudaMemcpyAsync((char*)da + r0 * k * 2, a + r0 * k, nr * k * 2, cudaMemcpyHostToDevice, e->h2d_stream);
      cudaEventRecord(ev[2 * p], e->h2d_stream);
      cudaStreamWaitEvent(e->stream, ev[2 * p], 0);
      GemmArgs g{};
      g.a = (char*)da + r0 * k * 2; g.b = db; g.c = (char*)dc + r0 * n * 2;
      g.in_bf16 = 1; g.out_bf16 = 1;
      g.m = nr; g.n = n; g.k = k;
      g.lda = k; g.ldb = n; g.ldc = n;
      g.a_trans = 0; g.b_trans = 0; g.batch = 1; g.batches_dev = nullptr;
      st = run_gemm(e, g, nullptr, "matmul_host_bf16");
      if (st) break;
      cudaEventRecord(ev[2 * p + 1], e->stream);
      cudaStreamWaitEvent(e->d2h_stream, ev[2 * p + 1], 0);
      if (ce == cudaSuccess) ce = cudaMemcpyAsync(out + r0 * n, (char*)dc + r0 * n * 2, nr * n * 2, cudaMemcpyDeviceToHost, e->d2h_stream);
    }
    if (!st && ce != cudaSuccess) st = e->cuda_fail(ce, "matmul_host_bf16: copy");
    // everything in flight ends before the blocks go back to the pool
    cudaStreamSynchronize(e->h2d_stream);
    cudaStreamSynchronize(e->d2h_stream);
    const int ws = e->wait();
    if (!st) st = ws;
    if (!st) { e->traffic.bytes_h2d += (m * k + k * n) * 2; e->traffic.bytes_d2h += m * n * 2; }
  }
  for (auto x : ev) if (x) cudaEventDestroy(x);
  if (da) e->release(da, ga);
  if (db) e->release(db, gb);
  if (dc) e->release(dc, gc);
  return st;
}

int32_t b200_matmul_batched(b200_engine* e, b200_buffer a, b200_buffer b, const b200_block* ab, const b200_block* bb,
                            uint64_t items, const uint64_t mkn[3], const b200_batched_layout* layout,
                            int32_t out_bf16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr;
  int st = e->need(a, &A, "matmul_batched");
  if (!st) st = e->need(b, &B, "matmul_batched");
  if (st) return st;
  const bool abf = A->elem == B200_BF16, bbf = B->elem == B200_BF16;
  if ((A->elem != B200_F32 && !abf) || (B->elem != B200_F32 && !bbf) || abf != bbf)
    return e->fail(B200_UNSUPPORTED, "matmul_batched: operands must both be F32 or both BF16");
  const uint64_t m = mkn[0], k = mkn[1], n = mkn[2];
  const bool stacked = !layout || layout->stacked;
  const uint64_t step = stacked ? m : ((m + 31) / 32) * 32;  // server.rs:3749-3754
  std::vector<GemmBatch> bt(items);
  for (uint64_t i = 0; i < items; ++i) {
    const b200_block &x = ab[i], &y = bb[i];
    const uint64_t ar = x.transposed ? k : m, ac = x.transposed ? m : k;
    const uint64_t br = y.transposed ? n : k, bc = y.transposed ? k : n;
    if (x.at[0] + ar > A->rows || x.at[1] + ac > A->cols || y.at[0] + br > B->rows || y.at[1] + bc > B->cols)
      return e->fail(B200_UNSUPPORTED, "matmul_batched: item %llu's block lies outside its buffer", (unsigned long long)i);
    bt[i].a_off = x.at[0] * A->cols + x.at[1];
    bt[i].b_off = y.at[0] * B->cols + y.at[1];
    bt[i].c_off = i * step * n;
    bt[i].a_trans = x.transposed; bt[i].b_trans = y.transposed;
  }
  Buf* C = nullptr;
  st = e->new_buffer(items * step, n, out_bf16 ? B200_BF16 : B200_F32, out, &C);
  if (st) return st;
  A = e->get(a); B = e->get(b);
  if ((!stacked && step != m) || k == 0) cudaMemsetAsync(C->ptr, 0, items * step * n * elem_bytes(C->elem), e->stream);
  if (items == 1 && k) {
    // One item is one plain product on the item's blocks: the block offsets move the operands' bases and the
    // item's transposed flags are the product's, so every kernel sees what it sees for `matmul_dram` (the
    // kernels key "batched" on more than one item and would otherwise drop the item's offsets and flags).
    const uint64_t eb = elem_bytes(A->elem);
    GemmArgs g{};
    g.a = (const char*)A->ptr + bt[0].a_off * eb; g.b = (const char*)B->ptr + bt[0].b_off * eb; g.c = C->ptr;
    g.in_bf16 = abf; g.out_bf16 = out_bf16;
    g.m = m; g.n = n; g.k = k;
    g.lda = A->cols; g.ldb = B->cols; g.ldc = n;
    g.a_trans = bt[0].a_trans; g.b_trans = bt[0].b_trans;
    g.batch = 1; g.batches_dev = nullptr;
    st = run_gemm(e, g, nullptr, "matmul_batched");
    if (st) { e->drop(*out); return st; }
  } else if (items && k) {
    void* dev = nullptr;
    uint64_t got = 0;
    st = e->to_device(bt.data(), items * sizeof(GemmBatch), &dev, &got);
    if (st) { e->drop(*out); return st; }
    GemmArgs g{};
    g.a = A->ptr; g.b = B->ptr; g.c = C->ptr;
    g.in_bf16 = abf; g.out_bf16 = out_bf16;
    g.m = m; g.n = n; g.k = k;
    g.lda = A->cols; g.ldb = B->cols; g.ldc = n;
    g.batch = items; g.batches_dev = (const GemmBatch*)dev;
    st = run_gemm(e, g, bt.data(), "matmul_batched");
    e->release(dev, got);
    if (st) { e->drop(*out); return st; }
  }
  set_dims(out_dims, items * step, n);
  return B200_OK;
}

// ---- element-wise ----------------------------------------------------------------
int32_t b200_eltwise(b200_engine* e, const b200_eltwise_op* op, b200_buffer a, b200_buffer b, b200_buffer c,
                     int32_t out_bf16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr, *C = nullptr;
  int st = e->need(a, &A, "eltwise");
  if (!st && b) st = e->need(b, &B, "eltwise");
  if (!st && c) st = e->need(c, &C, "eltwise");
  if (st) return st;
  Mat ma = mat_of(A), mb, mc;
  if (B) mb = mat_of(B);
  if (C) mc = mat_of(C);
  return run_eltwise(e, op, ma, B ? &mb : nullptr, C ? &mc : nullptr, out_bf16, out, out_dims);
}

int32_t b200_eltwise_blocks(b200_engine* e, const b200_eltwise_op* op, const b200_block_arg* a, const b200_block_arg* b,
                            const b200_block_arg* c, int32_t out_bf16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Mat ma, mb, mc;
  int st = mat_of_block(e, a, &ma, "eltwise_blocks");
  if (!st && b) st = mat_of_block(e, b, &mb, "eltwise_blocks");
  if (!st && c) st = mat_of_block(e, c, &mc, "eltwise_blocks");
  if (st) return st;
  return run_eltwise(e, op, ma, b ? &mb : nullptr, c ? &mc : nullptr, out_bf16, out, out_dims);
}

int32_t b200_cast_float(b200_engine* e, b200_buffer a, int32_t to_bf16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "cast_float");
  if (st) return st;
  const int want_in = to_bf16 ? B200_F32 : B200_BF16;
  if (A->elem != want_in) return e->fail(B200_UNSUPPORTED, "cast_float: source elem %d", A->elem);
  const uint64_t rows = A->rows, cols = A->cols;
  const void* src = A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(rows, cols, to_bf16 ? B200_BF16 : B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_cast(src, O->ptr, rows * cols, to_bf16, e->stream), "cast_float");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

// server.rs:141 `cast_bfp(id, format)`: F32 (or BF16) -> BFP8 storage (`format` 8), or BFP8 widened (`format` 0: to F32,
// the trait's `None`; -16: to BF16, which holds every decoded value exactly).
int32_t b200_cast_bfp(b200_engine* e, b200_buffer a, int32_t format, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "cast_bfp", true);
  if (st) return st;
  const uint64_t rows = A->rows, cols = A->cols;
  Buf* O = nullptr;
  if (format == 8) {
    if (A->elem != B200_F32 && A->elem != B200_BF16) return e->fail(B200_UNSUPPORTED, "cast_bfp: source elem %d is not F32 or BF16", A->elem);
    if (cols % 16) return e->fail(B200_UNSUPPORTED, "cast_bfp: %llu columns are not whole groups of sixteen", (unsigned long long)cols);
    st = e->new_buffer(rows, cols, B200_BFP8, out, &O);
    if (st) return st;
    A = e->get(a);
    uint8_t* datums = (uint8_t*)O->ptr;
    st = e->launched(launch_bfp8_encode(A->ptr, A->elem == B200_BF16, rows, cols, datums, datums + rows * cols, e->stream), "cast_bfp");
  } else if (format == 0 || format == -16) {
    if (A->elem != B200_BFP8) return e->fail(B200_UNSUPPORTED, "cast_bfp: buffer %llu is not BFP8 storage", (unsigned long long)a);
    st = e->new_buffer(rows, cols, format == 0 ? B200_F32 : B200_BF16, out, &O);
    if (st) return st;
    A = e->get(a);
    const uint8_t* datums = (const uint8_t*)A->ptr;
    st = e->launched(launch_bfp8_decode(datums, datums + rows * cols, rows, cols, O->ptr, format != 0, e->stream), "cast_bfp");
  } else {
    return e->fail(B200_UNSUPPORTED, "cast_bfp: format %d (8 stores BFP8, 0 widens to F32, -16 to BF16; BFP4 and BFP2 are not kept by this engine)", format);
  }
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

// The stored bytes of a BFP8 buffer, as they lie: rows * cols datums, then rows * cols / 16 exponents.
int32_t b200_download_bfp(b200_engine* e, b200_buffer id, uint8_t* datums, uint8_t* exponents, uint64_t capacity_datums) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "download_bfp inside a trace capture");
  Buf* A = nullptr;
  int st = e->need(id, &A, "download_bfp", true);
  if (st) return st;
  if (A->elem != B200_BFP8) return e->fail(B200_UNSUPPORTED, "download_bfp: buffer %llu is not BFP8 storage", (unsigned long long)id);
  const uint64_t n = A->rows * A->cols;
  if (capacity_datums < n) return e->fail(B200_UNSUPPORTED, "download_bfp: %llu datums into room for %llu", (unsigned long long)n, (unsigned long long)capacity_datums);
  if (n) {
    cudaError_t ce = cudaMemcpyAsync(datums, A->ptr, n, cudaMemcpyDeviceToHost, e->stream);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(exponents, (const uint8_t*)A->ptr + n, n / 16, cudaMemcpyDeviceToHost, e->stream);
    if (ce != cudaSuccess) return e->cuda_fail(ce, "download_bfp");
  }
  e->traffic.bytes_d2h += n + n / 16;
  e->traffic.d2h_calls++;
  return e->wait();
}

int32_t b200_rope_blocks(b200_engine* e, const b200_block_arg* x, const b200_block_arg* cs, const b200_block_arg* sn,
                         uint64_t head, int32_t out_bf16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Mat mx, mc, ms;
  int st = mat_of_block(e, x, &mx, "rope");
  if (!st) st = mat_of_block(e, cs, &mc, "rope");
  if (!st) st = mat_of_block(e, sn, &ms, "rope");
  if (st) return st;
  if (head == 0 || head % 2 || mx.cols % head)
    return e->fail(B200_UNSUPPORTED, "rope: %llu columns are not heads of %llu", (unsigned long long)mx.cols, (unsigned long long)head);
  auto table_ok = [&](const Mat& t) {
    return (t.cols == head || t.cols == mx.cols) && t.rows > 0 && mx.rows % t.rows == 0;
  };
  if (!table_ok(mc) || !table_ok(ms)) return e->fail(B200_UNSUPPORTED, "rope: a table's shape does not meet x's");
  Buf* O = nullptr;
  st = e->new_buffer(mx.rows, mx.cols, out_bf16 ? B200_BF16 : B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_rope(mx, mc, ms, head, O->ptr, mx.cols, out_bf16, mx.rows, mx.cols, e->stream), "rope");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, mx.rows, mx.cols);
  return B200_OK;
}

// ---- reductions ------------------------------------------------------------------
int32_t b200_reduce(b200_engine* e, b200_buffer a, int32_t op, int32_t axis, uint32_t then_kind, uint32_t then_bits,
                    b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "reduce");
  if (st) return st;
  if (op < 0 || op > B200_MAX_I32 || (axis != 0 && axis != 1)) return e->fail(B200_UNSUPPORTED, "reduce: op %d axis %d", op, axis);
  switch (then_kind) {
    case 0: case kind::NEG: case kind::ABS: case kind::SIGN: case kind::RELU: case kind::CLAMP_MIN:
    case kind::CLAMP_MAX: case kind::INT_ABS: break;
    default: return e->fail(B200_UNSUPPORTED, "reduce: kind %#x is not an exact unary finishing kind", then_kind);
  }
  const int oelem = (op == B200_ALL || op == B200_ANY) ? B200_BOOL : (op >= B200_SUM_I32 ? B200_I32 : B200_F32);
  if (A->elem == B200_BF16 && oelem != B200_F32) return e->fail(B200_UNSUPPORTED, "reduce: an integer fold of a BF16 tensor");
  const uint64_t rows = A->rows, cols = A->cols;
  const void* src = A->ptr;
  const int bf = A->elem == B200_BF16;
  const uint64_t orows = axis == 0 ? 1 : rows, ocols = axis == 0 ? cols : 1;
  Buf* O = nullptr;
  st = e->new_buffer(orows, ocols, oelem, out, &O);
  if (st) return st;
  st = e->launched(launch_reduce(src, bf, rows, cols, op, axis, then_kind, then_bits, O->ptr, e->stream), "reduce");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, orows, ocols);
  return B200_OK;
}
int32_t b200_sum_rows(b200_engine* e, b200_buffer a, b200_buffer* out, uint64_t out_dims[2]) {
  return b200_reduce(e, a, B200_SUM, B200_ROWS, 0, 0, out, out_dims);
}
int32_t b200_full_sum(b200_engine* e, b200_buffer a, int32_t mean, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "full_sum");
  if (st) return st;
  if (A->elem != B200_F32) return e->fail(B200_UNSUPPORTED, "full_sum: F32 only");
  const float* src = (const float*)A->ptr;
  const uint64_t n = A->rows * A->cols;
  Buf* O = nullptr;
  st = e->new_buffer(1, 1, B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_full_sum(src, n, mean, e->full_scratch, (float*)O->ptr, e->stream), "full_sum", 1);
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, 1, 1);
  return B200_OK;
}
int32_t b200_full_reduce(b200_engine* e, const float* values, const uint64_t dims[2], int32_t mean, float* out) {
  b200_buffer ia = 0, io = 0;
  uint64_t d[2];
  int st = b200_upload_f32(e, values, dims[0], dims[1], &ia);
  if (!st) st = b200_full_sum(e, ia, mean, &io, d);
  if (!st) st = b200_download_f32(e, io, out, 1);
  b200_free(e, ia); b200_free(e, io);
  return st;
}

static int softmax_any(b200_engine* e, b200_buffer x, b200_buffer mask, float scale, int log_form, int out_bf16,
                       b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *X = nullptr, *M = nullptr;
  int st = e->need(x, &X, "softmax_rows");
  if (!st && mask) st = e->need(mask, &M, "softmax_rows");
  if (st) return st;
  if (X->elem != B200_F32) return e->fail(B200_UNSUPPORTED, "softmax_rows: F32 scores only");
  if (M && (M->elem != B200_BOOL || M->cols != X->cols || M->rows == 0 || X->rows % M->rows))
    return e->fail(B200_UNSUPPORTED, "softmax_rows: mask [%llu,%llu] does not meet [%llu,%llu]", (unsigned long long)M->rows,
                   (unsigned long long)M->cols, (unsigned long long)X->rows, (unsigned long long)X->cols);
  const uint64_t rows = X->rows, cols = X->cols;
  const float* xs = (const float*)X->ptr;
  const uint32_t* ms = M ? (const uint32_t*)M->ptr : nullptr;
  const uint64_t mrows = M ? M->rows : 1;
  Buf* O = nullptr;
  st = e->new_buffer(rows, cols, out_bf16 ? B200_BF16 : B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_softmax_rows(xs, ms, mrows, scale, log_form, O->ptr, out_bf16, rows, cols, e->stream), "softmax_rows");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}
int32_t b200_softmax_rows(b200_engine* e, b200_buffer x, b200_buffer mask, float scale, b200_buffer* out, uint64_t out_dims[2]) {
  return softmax_any(e, x, mask, scale, 0, 0, out, out_dims);
}
int32_t b200_softmax_rows_as(b200_engine* e, b200_buffer x, b200_buffer mask, float scale, int32_t out_bf16, b200_buffer* out,
                             uint64_t out_dims[2]) {
  return softmax_any(e, x, mask, scale, 0, out_bf16, out, out_dims);
}
int32_t b200_log_softmax_rows(b200_engine* e, b200_buffer x, b200_buffer* out, uint64_t out_dims[2]) {
  return softmax_any(e, x, 0, 1.0f, 1, 0, out, out_dims);
}

int32_t b200_rms(b200_engine* e, b200_buffer a, float eps, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "rms");
  if (st) return st;
  if (A->elem != B200_F32) return e->fail(B200_UNSUPPORTED, "rms: F32 only");
  const uint64_t rows = A->rows, cols = A->cols;
  const float* src = (const float*)A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(rows, 1, B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_rms(src, rows, cols, eps, (float*)O->ptr, e->stream), "rms");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, 1);
  return B200_OK;
}

static bool is_float(const Buf* b) { return b->elem == B200_F32 || b->elem == B200_BF16; }

int32_t b200_rms_norm(b200_engine* e, b200_buffer a, b200_buffer gamma, float eps, int32_t out_bf16, b200_buffer* out,
                      uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *G = nullptr;
  int st = e->need(a, &A, "rms_norm");
  if (!st && gamma) st = e->need(gamma, &G, "rms_norm");
  if (st) return st;
  if (!is_float(A) || (G && (!is_float(G) || G->rows != 1 || G->cols != A->cols)))
    return e->fail(B200_UNSUPPORTED, "rms_norm: gamma must be [1, cols] floats");
  const uint64_t rows = A->rows, cols = A->cols;
  const void* src = A->ptr; const int abf = A->elem == B200_BF16;
  const void* gp = G ? G->ptr : nullptr; const int gbf = G ? G->elem == B200_BF16 : 0;
  Buf* O = nullptr;
  st = e->new_buffer(rows, cols, out_bf16 ? B200_BF16 : B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_rms_norm(src, abf, nullptr, 0, gp, gbf, eps, nullptr, 0, O->ptr, out_bf16, rows, cols, e->stream), "rms_norm");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_add_rms_norm(b200_engine* e, b200_buffer a, b200_buffer b, b200_buffer gamma, float eps, b200_buffer out[2],
                          uint64_t out_dims[2]) {
  return b200_add_rms_norm_as(e, a, b, gamma, eps, 0, out, out_dims);
}

int32_t b200_add_rms_norm_as(b200_engine* e, b200_buffer a, b200_buffer b, b200_buffer gamma, float eps, int32_t norm_bf16,
                             b200_buffer out[2], uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *A = nullptr, *B = nullptr, *G = nullptr;
  int st = e->need(a, &A, "add_rms_norm");
  if (!st) st = e->need(b, &B, "add_rms_norm");
  if (!st && gamma) st = e->need(gamma, &G, "add_rms_norm");
  if (st) return st;
  if (!is_float(A) || !is_float(B) || A->rows != B->rows || A->cols != B->cols ||
      (G && (!is_float(G) || G->rows != 1 || G->cols != A->cols)))
    return e->fail(B200_UNSUPPORTED, "add_rms_norm: operand shapes do not meet");
  const uint64_t rows = A->rows, cols = A->cols;
  const int abf = A->elem == B200_BF16, bbf = B->elem == B200_BF16;
  const int obf = abf && bbf;  // results in the operands' type
  const void *ap = A->ptr, *bp = B->ptr, *gp = G ? G->ptr : nullptr;
  const int gbf = G ? G->elem == B200_BF16 : 0;
  Buf *S = nullptr, *N = nullptr;
  st = e->new_buffer(rows, cols, obf ? B200_BF16 : B200_F32, &out[0], &S);
  if (st) return st;
  void* sp = S->ptr;
  const int nbf = obf || norm_bf16;   // the norm rounded once to BF16 where asked
  st = e->new_buffer(rows, cols, nbf ? B200_BF16 : B200_F32, &out[1], &N);
  if (st) { e->drop(out[0]); return st; }
  st = e->launched(launch_rms_norm(ap, abf, bp, bbf, gp, gbf, eps, sp, obf, N->ptr, nbf, rows, cols, e->stream), "add_rms_norm");
  if (st) { e->drop(out[0]); e->drop(out[1]); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_argmax_row(b200_engine* e, b200_buffer a, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "argmax_row");
  if (st) return st;
  if (A->elem != B200_F32) return e->fail(B200_UNSUPPORTED, "argmax_row: F32 only");
  if (A->cols == 0 || A->cols > (1ull << 31)) return e->fail(B200_UNSUPPORTED, "argmax_row: %llu columns", (unsigned long long)A->cols);
  const uint64_t rows = A->rows, cols = A->cols;
  const float* src = (const float*)A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(rows, 1, B200_I32, out, &O);
  if (st) return st;
  st = e->launched(launch_argmax_rows(src, rows, cols, (int32_t*)O->ptr, e->stream), "argmax_row");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, 1);
  return B200_OK;
}

// ---- indexing ----------------------------------------------------------------------
int32_t b200_select_rows(b200_engine* e, b200_buffer table, b200_buffer indices, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *T = nullptr, *I = nullptr;
  int st = e->need(table, &T, "select_rows");
  if (!st) st = index_buf(e, indices, &I, "select_rows");
  if (st) return st;
  const uint64_t n = I->rows * I->cols, cols = T->cols, trows = T->rows;
  const int elem = T->elem;
  const void* tp = T->ptr; const int32_t* ip = (const int32_t*)I->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(n, cols, elem, out, &O);
  if (st) return st;
  st = e->launched(launch_select_rows(tp, trows, cols, (int)elem_bytes(elem), ip, n, O->ptr, e->d_err, e->stream), "select_rows");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, n, cols);
  return B200_OK;
}

int32_t b200_pick_columns(b200_engine* e, b200_buffer input, b200_buffer indices, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *X = nullptr, *I = nullptr;
  int st = e->need(input, &X, "pick_columns");
  if (!st) st = index_buf(e, indices, &I, "pick_columns");
  if (st) return st;
  if (elem_bytes(X->elem) != 4 || I->rows * I->cols != X->rows)
    return e->fail(B200_UNSUPPORTED, "pick_columns: [%llu,%llu] with %llu indices", (unsigned long long)X->rows,
                   (unsigned long long)X->cols, (unsigned long long)(I->rows * I->cols));
  const uint64_t rows = X->rows, cols = X->cols;
  const int elem = X->elem;
  const uint32_t* xp = (const uint32_t*)X->ptr; const int32_t* ip = (const int32_t*)I->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(rows, 1, elem, out, &O);
  if (st) return st;
  st = e->launched(launch_pick_columns(xp, rows, cols, ip, (uint32_t*)O->ptr, e->d_err, e->stream), "pick_columns");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, 1);
  return B200_OK;
}

int32_t b200_scatter_add_columns(b200_engine* e, b200_buffer t, b200_buffer indices, b200_buffer value, b200_buffer* out,
                                 uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *T = nullptr, *I = nullptr, *V = nullptr;
  int st = e->need(t, &T, "scatter_add_columns");
  if (!st) st = index_buf(e, indices, &I, "scatter_add_columns");
  if (!st) st = e->need(value, &V, "scatter_add_columns");
  if (st) return st;
  if (T->elem != B200_F32 || V->elem != B200_F32 || I->rows * I->cols != T->rows || V->rows * V->cols != T->rows)
    return e->fail(B200_UNSUPPORTED, "scatter_add_columns: shapes do not meet");
  const uint64_t rows = T->rows, cols = T->cols;
  Buf* O = nullptr;
  st = copy_of(e, T, out, &O);
  if (st) return st;
  I = e->get(indices); V = e->get(value);
  st = e->launched(launch_scatter_add_columns((float*)O->ptr, rows, cols, (const int32_t*)I->ptr, (const float*)V->ptr, e->d_err, e->stream),
                   "scatter_add_columns");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_select_add_rows(b200_engine* e, b200_buffer t, b200_buffer indices, b200_buffer value, b200_buffer* out,
                             uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *T = nullptr, *I = nullptr, *V = nullptr;
  int st = e->need(t, &T, "select_add_rows");
  if (!st) st = index_buf(e, indices, &I, "select_add_rows");
  if (!st) st = e->need(value, &V, "select_add_rows");
  if (st) return st;
  const uint64_t n = I->rows * I->cols;
  if (T->elem != B200_F32 || V->elem != B200_F32 || V->rows != n || V->cols != T->cols)
    return e->fail(B200_UNSUPPORTED, "select_add_rows: shapes do not meet");
  const uint64_t rows = T->rows, cols = T->cols;
  Buf* O = nullptr;
  st = copy_of(e, T, out, &O);
  if (st) return st;
  I = e->get(indices); V = e->get(value);
  st = e->launched(launch_select_add_rows((float*)O->ptr, rows, cols, (const int32_t*)I->ptr, n, (const float*)V->ptr, e->d_err, e->stream),
                   "select_add_rows");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_rows_add(b200_engine* e, b200_buffer t, const uint64_t* indices, uint64_t n, b200_buffer value, b200_buffer* out,
                      uint64_t out_dims[2]) {
  // The host's index list goes to the device as a block list does (kept by content, or a copy node of an
  // open capture), so the call is as capturable as `select_add_rows` itself.
  cudaSetDevice(e->device);
  Buf *T = nullptr, *V = nullptr;
  int st = e->need(t, &T, "rows_add");
  if (!st) st = e->need(value, &V, "rows_add");
  if (st) return st;
  if (T->elem != B200_F32 || V->elem != B200_F32 || V->rows != n || V->cols != T->cols)
    return e->fail(B200_UNSUPPORTED, "rows_add: shapes do not meet");
  const uint64_t rows = T->rows, cols = T->cols;
  std::vector<int32_t> idx(n);
  for (uint64_t i = 0; i < n; ++i) idx[i] = indices[i] > 0x7fffffffull ? -1 : (int32_t)indices[i];   // outside every table: DOMAIN
  Buf* O = nullptr;
  st = copy_of(e, T, out, &O);
  if (st) return st;
  V = e->get(value);
  if (n) {
    void* dev = nullptr; uint64_t got = 0;
    st = e->to_device(idx.data(), n * sizeof(int32_t), &dev, &got);
    if (st) { e->drop(*out); return st; }
    st = e->launched(launch_select_add_rows((float*)O->ptr, rows, cols, (const int32_t*)dev, n, (const float*)V->ptr, e->d_err, e->stream),
                     "rows_add");
    e->release(dev, got);
    if (st) { e->drop(*out); return st; }
  }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_assign_rows(b200_engine* e, b200_buffer t, b200_buffer value, const uint64_t* pairs, uint64_t n, b200_buffer* out,
                         uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *T = nullptr, *V = nullptr;
  int st = e->need(t, &T, "assign_rows");
  if (!st) st = e->need(value, &V, "assign_rows");
  if (st) return st;
  if (T->elem != V->elem || T->cols != V->cols) return e->fail(B200_UNSUPPORTED, "assign_rows: value does not meet the table");
  for (uint64_t i = 0; i < n; ++i)
    if (pairs[2 * i] >= T->rows || pairs[2 * i + 1] >= V->rows) return e->fail(B200_DOMAIN, "assign_rows: DOMAIN: pair %llu names a row outside", (unsigned long long)i);
  const uint64_t rows = T->rows, cols = T->cols;
  const int eb = (int)elem_bytes(T->elem);
  Buf* O = nullptr;
  st = copy_of(e, T, out, &O);
  if (st) return st;
  void* op = O->ptr;
  V = e->get(value);
  const void* vp = V->ptr;
  if (n) {
    void* dev = nullptr; uint64_t got = 0;
    st = e->to_device(pairs, n * 16, &dev, &got);
    if (st) { e->drop(*out); return st; }
    st = e->launched(launch_assign_rows(op, vp, cols, eb, (const uint64_t*)dev, n, e->stream), "assign_rows");
    e->release(dev, got);
    if (st) { e->drop(*out); return st; }
  }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_scatter_rows(b200_engine* e, b200_buffer table, b200_buffer indices, b200_buffer values, int32_t column,
                          b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *T = nullptr, *I = nullptr, *V = nullptr;
  int st = e->need(table, &T, "scatter_rows");
  if (!st) st = index_buf(e, indices, &I, "scatter_rows");
  if (!st) st = e->need(values, &V, "scatter_rows");
  if (st) return st;
  const uint64_t n = I->rows * I->cols;
  if ((column ? I->cols : I->rows) != 1 || elem_bytes(T->elem) != 4 || V->elem != T->elem || V->rows != n || V->cols != T->cols)
    return e->fail(B200_UNSUPPORTED, "scatter_rows: shapes do not meet");
  const uint64_t rows = T->rows, cols = T->cols;
  Buf* O = nullptr;
  st = copy_of(e, T, out, &O);
  if (st) return st;
  I = e->get(indices); V = e->get(values);
  st = e->launched(launch_scatter_rows((uint32_t*)O->ptr, rows, cols, (const int32_t*)I->ptr, n, (const uint32_t*)V->ptr, e->d_err, e->stream),
                   "scatter_rows");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_scatter_rows_into(b200_engine* e, b200_buffer table, b200_buffer indices, const b200_block_arg* values, int32_t column) {
  cudaSetDevice(e->device);
  Buf *T = nullptr, *I = nullptr, *V = nullptr;
  int st = e->need(table, &T, "scatter_rows_into");
  if (!st) st = index_buf(e, indices, &I, "scatter_rows_into");
  if (!st) st = e->need(values->id, &V, "scatter_rows_into");
  if (st) return st;
  const uint64_t n = I->rows * I->cols;
  const bool narrow = T->elem == B200_BF16 && V->elem == B200_F32;   // F32 rows rounded once into a BF16 table
  if ((column ? I->cols : I->rows) != 1 || (V->elem != T->elem && !narrow) || values->dims[0] != n || values->dims[1] != T->cols ||
      values->at[0] + values->dims[0] > V->rows || values->at[1] + values->dims[1] > V->cols)
    return e->fail(B200_UNSUPPORTED, "scatter_rows_into: shapes do not meet");
  const int eb = (int)elem_bytes(T->elem);
  const char* vp = (const char*)V->ptr + (values->at[0] * V->cols + values->at[1]) * elem_bytes(V->elem);
  return e->launched(launch_scatter_rows_into(T->ptr, T->rows, T->cols, narrow ? -2 : eb, (const int32_t*)I->ptr, n, vp, V->cols, e->d_err,
                                              e->stream),
                     "scatter_rows_into");
}

int32_t b200_reshape(b200_engine* e, b200_buffer a, uint64_t rows, uint64_t cols, b200_buffer* out, uint64_t out_dims[2]) {
  Buf* A = nullptr;
  int st = e->need(a, &A, "reshape");
  if (st) return st;
  if (rows * cols != A->rows * A->cols)
    return e->fail(B200_UNSUPPORTED, "reshape: [%llu, %llu] as [%llu, %llu]", (unsigned long long)A->rows, (unsigned long long)A->cols,
                   (unsigned long long)rows, (unsigned long long)cols);
  Buf v;
  v.ptr = A->ptr;
  v.rows = rows; v.cols = cols; v.elem = A->elem; v.parent = a;
  A->views++;
  *out = e->next_id++;
  e->bufs.emplace(*out, v);
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_gather_indexed(b200_engine* e, b200_buffer input, b200_buffer indices, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *X = nullptr, *I = nullptr;
  int st = e->need(input, &X, "gather_indexed");
  if (!st) st = index_buf(e, indices, &I, "gather_indexed");
  if (st) return st;
  if (elem_bytes(X->elem) != 4 || I->rows != X->rows) return e->fail(B200_UNSUPPORTED, "gather_indexed: shapes do not meet");
  const uint64_t rows = X->rows, cols = X->cols, icols = I->cols;
  const int elem = X->elem;
  const uint32_t* xp = (const uint32_t*)X->ptr; const int32_t* ip = (const int32_t*)I->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(rows, icols, elem, out, &O);
  if (st) return st;
  st = e->launched(launch_gather_indexed(xp, rows, cols, ip, icols, (uint32_t*)O->ptr, e->d_err, e->stream), "gather_indexed");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, icols);
  return B200_OK;
}

int32_t b200_gather_rows(b200_engine* e, const b200_buffer* sources, uint64_t n_sources, const uint64_t* pairs, uint64_t n_rows,
                         uint64_t cols, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  if (n_sources == 0) return e->fail(B200_UNSUPPORTED, "gather_rows: no source");
  std::vector<Buf*> src(n_sources);
  for (uint64_t i = 0; i < n_sources; ++i) {
    int st = e->need(sources[i], &src[i], "gather_rows");
    if (st) return st;
    if (src[i]->cols != cols || src[i]->elem != src[0]->elem) return e->fail(B200_UNSUPPORTED, "gather_rows: source %llu does not have %llu columns of the first's type", (unsigned long long)i, (unsigned long long)cols);
  }
  const int elem = src[0]->elem;
  const uint64_t eb = elem_bytes(elem);
  std::vector<const void*> ptrs(n_rows);
  for (uint64_t i = 0; i < n_rows; ++i) {
    const uint64_t s = pairs[2 * i], r = pairs[2 * i + 1];
    if (s >= n_sources || r >= src[s]->rows) return e->fail(B200_DOMAIN, "gather_rows: DOMAIN: row %llu names (%llu, %llu)", (unsigned long long)i, (unsigned long long)s, (unsigned long long)r);
    ptrs[i] = (const char*)src[s]->ptr + r * cols * eb;
  }
  Buf* O = nullptr;
  int st = e->new_buffer(n_rows, cols, elem, out, &O);
  if (st) return st;
  void* op = O->ptr;
  if (n_rows) {
    void* dev = nullptr; uint64_t got = 0;
    st = e->to_device(ptrs.data(), n_rows * sizeof(void*), &dev, &got);
    if (st) { e->drop(*out); return st; }
    st = e->launched(launch_gather_row_ptrs((const void* const*)dev, n_rows, cols, (int)eb, op, e->stream), "gather_rows");
    e->release(dev, got);
    if (st) { e->drop(*out); return st; }
  }
  set_dims(out_dims, n_rows, cols);
  return B200_OK;
}

int32_t b200_slice_rows(b200_engine* e, b200_buffer a, uint64_t first, uint64_t rows, b200_buffer* out, uint64_t out_dims[2]) {
  Buf* A = nullptr;
  int st = e->need(a, &A, "slice_rows");
  if (st) return st;
  if (first + rows > A->rows) return e->fail(B200_UNSUPPORTED, "slice_rows: rows %llu..%llu of %llu", (unsigned long long)first, (unsigned long long)(first + rows), (unsigned long long)A->rows);
  Buf v;
  v.ptr = (char*)A->ptr + first * A->cols * elem_bytes(A->elem);
  v.rows = rows; v.cols = A->cols; v.elem = A->elem; v.parent = a;
  A->views++;
  *out = e->next_id++;
  e->bufs.emplace(*out, v);
  set_dims(out_dims, rows, v.cols);
  return B200_OK;
}

int32_t b200_copy_blocks(b200_engine* e, b200_buffer a, const b200_block_move* moves, uint64_t n, const uint64_t dims[2],
                         b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "copy_blocks");
  if (st) return st;
  std::vector<MoveDev> mv(n);
  uint64_t area = 0, max_r = 0, max_c = 0;
  for (uint64_t i = 0; i < n; ++i) {
    const b200_block_move& m = moves[i];
    const uint64_t sr = m.transposed ? m.extent[1] : m.extent[0], sc = m.transposed ? m.extent[0] : m.extent[1];
    if (m.from[0] + sr > A->rows || m.from[1] + sc > A->cols || m.to[0] + m.extent[0] > dims[0] || m.to[1] + m.extent[1] > dims[1])
      return e->fail(B200_UNSUPPORTED, "copy_blocks: move %llu lies outside a tensor", (unsigned long long)i);
    mv[i] = MoveDev{m.from[0], m.from[1], m.to[0], m.to[1], m.extent[0], m.extent[1], m.transposed, 0};
    area += m.extent[0] * m.extent[1];
    max_r = std::max(max_r, m.extent[0]); max_c = std::max(max_c, m.extent[1]);
  }
  if (area != dims[0] * dims[1]) return e->fail(B200_UNSUPPORTED, "copy_blocks: the blocks do not cover the output exactly once");
  const int elem = A->elem;
  const uint64_t src_ld = A->cols;
  const void* sp = A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(dims[0], dims[1], elem, out, &O);
  if (st) return st;
  void* op = O->ptr;
  if (n) {
    void* dev = nullptr; uint64_t got = 0;
    st = e->to_device(mv.data(), n * sizeof(MoveDev), &dev, &got);
    if (st) { e->drop(*out); return st; }
    st = e->launched(launch_copy_blocks(sp, src_ld, op, dims[1], (int)elem_bytes(elem), (const MoveDev*)dev, n, max_r, max_c, e->stream), "copy_blocks");
    e->release(dev, got);
    if (st) { e->drop(*out); return st; }
  }
  set_dims(out_dims, dims[0], dims[1]);
  return B200_OK;
}

int32_t b200_attention_rows(b200_engine* e, const b200_buffer buffers[4], const b200_attention_item* items, uint64_t n_items,
                            const uint64_t dims[4], float scale, b200_buffer* out, uint64_t out_dims[2]) {
  return b200_attention_rows_as(e, buffers, items, n_items, dims, scale, 0, out, out_dims);
}

int32_t b200_attention_rows_as(b200_engine* e, const b200_buffer buffers[4], const b200_attention_item* items, uint64_t n_items,
                               const uint64_t dims[4], float scale, int32_t out_bf16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *Q = nullptr, *K = nullptr, *V = nullptr, *M = nullptr;
  int st = e->need(buffers[0], &Q, "attention_rows");
  if (!st) st = e->need(buffers[1], &K, "attention_rows");
  if (!st) st = e->need(buffers[2], &V, "attention_rows");
  if (!st) st = e->need(buffers[3], &M, "attention_rows");
  if (st) return st;
  const uint64_t m = dims[0], d = dims[1], l = dims[2], dv = dims[3];
  if (Q->elem != B200_F32) return e->fail(B200_UNSUPPORTED, "attention_rows: queries are F32");
  if ((K->elem != B200_F32 && K->elem != B200_BF16) || V->elem != K->elem)
    return e->fail(B200_UNSUPPORTED, "attention_rows: keys and values are both F32 or both BF16");
  if (M->elem != B200_BOOL) return e->fail(B200_UNSUPPORTED, "attention_rows: the mask is Bool");
  if (n_items == 0) return e->fail(B200_UNSUPPORTED, "attention_rows: no heads");
  if (M->rows != 1 || M->cols != l)
    return e->fail(B200_UNSUPPORTED, "attention_rows: a [%llu, %llu] mask for %llu positions",
                   (unsigned long long)M->rows, (unsigned long long)M->cols, (unsigned long long)l);
  if (m < 1 || m > 32 || d == 0 || l == 0 || dv == 0 || d % 32 || l % 32 || dv % 32 || l > (1ull << 30) || d > 8192 || dv > 8192)
    return e->fail(B200_UNSUPPORTED, "attention_rows: [m, d, l, dv] = [%llu, %llu, %llu, %llu] (1..32 rows, whole tiles along d, l and dv)",
                   (unsigned long long)m, (unsigned long long)d, (unsigned long long)l, (unsigned long long)dv);
  const int kv_bf16 = K->elem == B200_BF16;
  const uint64_t al = kv_bf16 ? 8 : 4;   // 16-byte pieces of a key or value row
  if (K->cols % al || V->cols % al)
    return e->fail(B200_UNSUPPORTED, "attention_rows: key and value buffers are a multiple of %llu columns wide", (unsigned long long)al);
  // Heads that share a key block and a value block (grouped-query attention) become one job of up
  // to 8 query rows, in the order the heads came.
  std::vector<AttnRow> rows;
  std::vector<AttnJob> jobs;
  std::map<std::pair<uint64_t, uint64_t>, std::vector<uint32_t>> groups;
  std::vector<std::pair<uint64_t, uint64_t>> order;
  rows.reserve(n_items * m);
  for (uint64_t i = 0; i < n_items; ++i) {
    const b200_attention_item& it = items[i];
    if (it.q[0] + m > Q->rows || it.q[1] + d > Q->cols || it.k[0] + l > K->rows || it.k[1] + d > K->cols ||
        it.v[0] + l > V->rows || it.v[1] + dv > V->cols)
      return e->fail(B200_UNSUPPORTED, "attention_rows: head %llu's blocks lie outside a tensor", (unsigned long long)i);
    if (it.k[1] % al || it.v[1] % al)
      return e->fail(B200_UNSUPPORTED, "attention_rows: head %llu's keys or values start at a column that is not a multiple of %llu",
                     (unsigned long long)i, (unsigned long long)al);
    const std::pair<uint64_t, uint64_t> key(it.k[0] * K->cols + it.k[1], it.v[0] * V->cols + it.v[1]);
    auto g = groups.find(key);
    if (g == groups.end()) { g = groups.emplace(key, std::vector<uint32_t>()).first; order.push_back(key); }
    for (uint64_t r = 0; r < m; ++r) {
      g->second.push_back((uint32_t)rows.size());
      rows.push_back(AttnRow{(it.q[0] + r) * Q->cols + it.q[1], (i * m + r) * dv});
    }
  }
  std::vector<AttnRow> sorted;
  sorted.reserve(rows.size());
  int widest = 1;
  for (const auto& key : order) {
    const std::vector<uint32_t>& members = groups[key];
    for (size_t at = 0; at < members.size(); at += 8) {
      const int take = (int)std::min<size_t>(8, members.size() - at);
      jobs.push_back(AttnJob{key.first, key.second, (int32_t)sorted.size(), take});
      for (int r = 0; r < take; ++r) sorted.push_back(rows[members[at + r]]);
      widest = std::max(widest, take);
    }
  }
  const uint64_t n_jobs = jobs.size();
  const int rt = attention_rows_tile(widest);
  int splits = 1, lc = (int)l;
  attention_rows_plan(n_jobs, rt, (int)l, /*sms: ask the device*/ 0, &splits, &lc);
  const float* qp = (const float*)Q->ptr; const void* kp = K->ptr; const void* vp = V->ptr; const uint32_t* mp = (const uint32_t*)M->ptr;
  const uint64_t k_ld = K->cols, v_ld = V->cols;
  Buf* O = nullptr;
  st = e->new_buffer(1, n_items * m * dv, out_bf16 ? B200_BF16 : B200_F32, out, &O);
  if (st) return st;
  void* op = O->ptr;
  std::vector<uint8_t> blob(n_jobs * sizeof(AttnJob) + sorted.size() * sizeof(AttnRow));
  memcpy(blob.data(), jobs.data(), n_jobs * sizeof(AttnJob));
  memcpy(blob.data() + n_jobs * sizeof(AttnJob), sorted.data(), sorted.size() * sizeof(AttnRow));
  void* dev = nullptr; uint64_t got = 0;
  st = e->to_device(blob.data(), blob.size(), &dev, &got);
  if (st) { e->drop(*out); return st; }
  void* scratch = nullptr; uint64_t sgot = 0;
  const size_t sfl = attention_rows_scratch_floats(n_jobs, rt, (int)dv, splits);
  if (sfl) {
    st = e->alloc(sfl * sizeof(float), &scratch, &sgot);
    if (st) { e->release(dev, got); e->drop(*out); return st; }
  }
  int launches = 0;
  const AttnJob* djobs = (const AttnJob*)dev;
  const AttnRow* drows = (const AttnRow*)((const uint8_t*)dev + n_jobs * sizeof(AttnJob));
  cudaError_t ce = launch_attention_rows(qp, kp, k_ld, vp, v_ld, kv_bf16, mp, djobs, drows, n_jobs, rt, (int)d, (int)l, (int)dv, scale,
                                         splits, lc, (float*)scratch, op, out_bf16 ? 1 : 0, &launches, e->stream);
  st = e->launched(ce, "attention_rows", launches > 0 ? launches : 1);
  if (scratch) e->release(scratch, sgot);
  e->release(dev, got);
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, 1, n_items * m * dv);
  return B200_OK;
}

int32_t b200_attention_blocks(b200_engine* e, b200_buffer q, b200_buffer k, b200_buffer v, const b200_attention_block* items,
                              uint64_t n_items, const uint64_t dims[4], float scale, int32_t causal, const uint64_t result_dims[2],
                              b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *Q = nullptr, *K = nullptr, *V = nullptr;
  int st = e->need(q, &Q, "attention_blocks");
  if (!st) st = e->need(k, &K, "attention_blocks");
  if (!st) st = e->need(v, &V, "attention_blocks");
  if (st) return st;
  const uint64_t sq = dims[0], d = dims[1], sk = dims[2], dv = dims[3];
  if (Q->elem != B200_BF16 || K->elem != B200_BF16 || V->elem != B200_BF16)
    return e->fail(B200_UNSUPPORTED, "attention_blocks: queries, keys and values are BF16");
  if (n_items == 0) return e->fail(B200_UNSUPPORTED, "attention_blocks: no blocks");
  const char* why = "";
  if (!attention_tc_supported(sq, d, sk, dv, scale, causal, &why))
    return e->fail(B200_UNSUPPORTED, "attention_blocks: [sq, d, sk, dv] = [%llu, %llu, %llu, %llu]: %s", (unsigned long long)sq,
                   (unsigned long long)d, (unsigned long long)sk, (unsigned long long)dv, why);
  const uint64_t o_rows = result_dims[0], o_cols = result_dims[1];
  const uint64_t lim = 1ull << 31;
  if (Q->cols % 8 || K->cols % 8 || V->cols % 8 || o_cols % 8 || o_rows == 0 || o_cols == 0 || Q->rows >= lim || K->rows >= lim ||
      V->rows >= lim || Q->cols >= lim || K->cols >= lim || V->cols >= lim)
    return e->fail(B200_UNSUPPORTED, "attention_blocks: buffer widths are multiples of 8 columns (and below 2^31)");
  std::vector<AttnBlockDev> host(n_items);
  uint64_t area = 0;
  for (uint64_t i = 0; i < n_items; ++i) {
    const b200_attention_block& it = items[i];
    if (it.q[0] + sq > Q->rows || it.q[1] + d > Q->cols || it.k[0] + sk > K->rows || it.k[1] + d > K->cols ||
        it.v[0] + sk > V->rows || it.v[1] + dv > V->cols || it.o[0] + sq > o_rows || it.o[1] + dv > o_cols)
      return e->fail(B200_UNSUPPORTED, "attention_blocks: block %llu lies outside a tensor", (unsigned long long)i);
    if (it.q[1] % 8 || it.k[1] % 8 || it.v[1] % 8 || it.o[1] % 8)
      return e->fail(B200_UNSUPPORTED, "attention_blocks: block %llu starts at a column that is not a multiple of 8", (unsigned long long)i);
    host[i] = AttnBlockDev{(int32_t)it.q[0], (int32_t)it.q[1], (int32_t)it.k[0], (int32_t)it.k[1], (int32_t)it.v[0], (int32_t)it.v[1],
                           0, 0, it.o[0] * o_cols + it.o[1]};
    area += sq * dv;
  }
  const void *qp = Q->ptr, *kp = K->ptr, *vp = V->ptr;
  const uint64_t qr = Q->rows, qc = Q->cols, kr = K->rows, kc = K->cols, vr = V->rows, vc = V->cols;
  Buf* O = nullptr;
  st = e->new_buffer(o_rows, o_cols, B200_BF16, out, &O);
  if (st) return st;
  void* op = O->ptr;
  if (area != o_rows * o_cols) {
    cudaError_t ce = cudaMemsetAsync(op, 0, o_rows * o_cols * 2, e->stream);
    if (ce != cudaSuccess) { e->drop(*out); return e->cuda_fail(ce, "attention_blocks"); }
  }
  void* dev = nullptr; uint64_t got = 0;
  st = e->to_device(host.data(), n_items * sizeof(AttnBlockDev), &dev, &got);
  if (st) { e->drop(*out); return st; }
  st = e->launched(launch_attention_tc(qp, qr, qc, kp, kr, kc, vp, vr, vc, (const AttnBlockDev*)dev, n_items, sq, d, sk, scale, causal,
                                       op, o_cols, e->d_err, e->stream), "attention_blocks");
  e->release(dev, got);
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, o_rows, o_cols);
  return B200_OK;
}

int32_t b200_repack(b200_engine* e, b200_buffer a, const uint64_t* pairs, const uint64_t dims[2], b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "repack");
  if (st) return st;
  const uint64_t n = dims[0] * dims[1];
  for (uint64_t i = 0; i < n; ++i)
    if (pairs[2 * i] >= A->rows || pairs[2 * i + 1] >= A->cols) return e->fail(B200_DOMAIN, "repack: DOMAIN: source %llu lies outside", (unsigned long long)i);
  const int elem = A->elem; const uint64_t ld = A->cols; const void* sp = A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(dims[0], dims[1], elem, out, &O);
  if (st) return st;
  void* op = O->ptr;
  if (n) {
    void* dev = nullptr; uint64_t got = 0;
    st = e->to_device(pairs, n * 16, &dev, &got);
    if (st) { e->drop(*out); return st; }
    st = e->launched(launch_repack(sp, ld, (int)elem_bytes(elem), (const uint64_t*)dev, n, op, e->stream), "repack");
    e->release(dev, got);
    if (st) { e->drop(*out); return st; }
  }
  set_dims(out_dims, dims[0], dims[1]);
  return B200_OK;
}

// ---- more movement and conversions: server.rs:95,137,309,317,578,705,779 -----------------------------
int32_t b200_repack_many(b200_engine* e, const b200_buffer* inputs, uint64_t n_inputs, const uint64_t* triples,
                         uint64_t n_triples, const uint64_t dims[2], b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  if (n_inputs == 0) return e->fail(B200_UNSUPPORTED, "repack_many: no inputs");
  if (dims[0] == 0 || dims[1] == 0) return e->fail(B200_UNSUPPORTED, "repack_many: an empty result");
  if (dims[0] * dims[1] != n_triples)     // crates/tt-kernels/src/tensor.rs:6803
    return e->fail(B200_UNSUPPORTED, "repack_many: %llu sources for a [%llu, %llu] result", (unsigned long long)n_triples,
                   (unsigned long long)dims[0], (unsigned long long)dims[1]);
  std::vector<Buf*> src(n_inputs);
  for (uint64_t i = 0; i < n_inputs; ++i) {
    int st = e->need(inputs[i], &src[i], "repack_many");
    if (st) return st;
    if (src[i]->elem != src[0]->elem) return e->fail(B200_UNSUPPORTED, "repack_many: input %llu is not of the first's element type", (unsigned long long)i);
  }
  const int elem = src[0]->elem;
  const uint64_t eb = elem_bytes(elem), n = dims[0] * dims[1];
  std::vector<uint64_t> addrs(n);
  for (uint64_t i = 0; i < n; ++i) {
    const uint64_t s = triples[3 * i], r = triples[3 * i + 1], c = triples[3 * i + 2];
    if (s >= n_inputs || r >= src[s]->rows || c >= src[s]->cols)
      return e->fail(B200_DOMAIN, "repack_many: DOMAIN: source %llu names (%llu, [%llu, %llu])", (unsigned long long)i,
                     (unsigned long long)s, (unsigned long long)r, (unsigned long long)c);
    addrs[i] = (uint64_t)(uintptr_t)((const char*)src[s]->ptr + (r * src[s]->cols + c) * eb);
  }
  Buf* O = nullptr;
  int st = e->new_buffer(dims[0], dims[1], elem, out, &O);
  if (st) return st;
  void* op = O->ptr;
  void* dev = nullptr; uint64_t got = 0;
  st = e->to_device(addrs.data(), n * 8, &dev, &got);
  if (st) { e->drop(*out); return st; }
  st = e->launched(launch_gather_addrs((const uint64_t*)dev, n, (int)eb, op, e->stream), "repack_many");
  e->release(dev, got);
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, dims[0], dims[1]);
  return B200_OK;
}

int32_t b200_select_taps(b200_engine* e, b200_buffer table, b200_buffer indices, int32_t zero_row, b200_buffer* out,
                         uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *T = nullptr, *I = nullptr;
  int st = e->need(table, &T, "select_taps");
  if (!st) st = index_buf(e, indices, &I, "select_taps");
  if (st) return st;
  const uint64_t taps = I->rows, n = I->cols, cols = T->cols, trows = T->rows;
  if (taps == 0 || cols == 0) return e->fail(B200_UNSUPPORTED, "select_taps: no taps or an empty table");
  const uint64_t out_cols = (taps - 1) * ((cols + 31) / 32 * 32) + cols;
  const int elem = T->elem;
  const void* tp = T->ptr; const int32_t* ip = (const int32_t*)I->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(n, out_cols, elem, out, &O);
  if (st) return st;
  st = e->launched(launch_select_taps(tp, trows, cols, (int)elem_bytes(elem), ip, taps, n, zero_row != 0, O->ptr, out_cols, e->d_err,
                                      e->stream), "select_taps");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, n, out_cols);
  return B200_OK;
}

int32_t b200_cast_block(b200_engine* e, const b200_block_arg* a, int32_t to_bf16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a->id, &A, "cast_block");
  if (st) return st;
  if (A->elem != (to_bf16 ? B200_F32 : B200_BF16)) return e->fail(B200_UNSUPPORTED, "cast_block: source elem %d", A->elem);
  const uint64_t rows = a->dims[0], cols = a->dims[1];
  if (a->at[0] + rows > A->rows || a->at[1] + cols > A->cols)
    return e->fail(B200_UNSUPPORTED, "cast_block: block [%llu, %llu] at [%llu, %llu] leaves its [%llu, %llu] buffer", (unsigned long long)rows,
                   (unsigned long long)cols, (unsigned long long)a->at[0], (unsigned long long)a->at[1], (unsigned long long)A->rows,
                   (unsigned long long)A->cols);
  const uint64_t ld = A->cols;
  const char* src = (const char*)A->ptr + (a->at[0] * ld + a->at[1]) * elem_bytes(A->elem);
  Buf* O = nullptr;
  st = e->new_buffer(rows, cols, to_bf16 ? B200_BF16 : B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_cast_block(src, ld, O->ptr, rows, cols, to_bf16 != 0, e->stream), "cast_block");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_cast_f16(b200_engine* e, b200_buffer a, int32_t to_f16, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "cast_f16");
  if (st) return st;
  if (A->elem != (to_f16 ? B200_F32 : B200_BF16))
    return e->fail(B200_UNSUPPORTED, "cast_f16: source elem %d (F32 narrows; two-byte storage widens)", A->elem);
  const uint64_t rows = A->rows, cols = A->cols;
  const void* src = A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(rows, cols, to_f16 ? B200_BF16 : B200_F32, out, &O);
  if (st) return st;
  st = e->launched(launch_cast_f16(src, O->ptr, rows * cols, to_f16 != 0, e->stream), "cast_f16");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_pow(b200_engine* e, b200_buffer x, int32_t exponent_kind, b200_buffer y, float scalar, b200_buffer* out,
                 uint64_t out_dims[2]) {
  b200_eltwise_op op{};
  if (exponent_kind == 1) { op.kind = kind::POW_S; op.scalar = scalar; return b200_eltwise(e, &op, x, 0, 0, 0, out, out_dims); }
  if (exponent_kind != 0 && exponent_kind != 2) return e->fail(B200_UNSUPPORTED, "pow: exponent kind %d", exponent_kind);
  Buf *X = nullptr, *Y = nullptr;
  int st = e->need(x, &X, "pow");
  if (!st) st = e->need(y, &Y, "pow");
  if (st) return st;
  if (Y->rows != X->rows || Y->cols != X->cols)     // crates/tt-kernels/src/session.rs:7746-7752
    return e->fail(B200_UNSUPPORTED, "pow: an exponent [%llu, %llu] for [%llu, %llu]", (unsigned long long)Y->rows, (unsigned long long)Y->cols,
                   (unsigned long long)X->rows, (unsigned long long)X->cols);
  if (Y->elem != (exponent_kind == 2 ? B200_I32 : B200_F32)) return e->fail(B200_UNSUPPORTED, "pow: exponent elem %d", Y->elem);
  op.kind = exponent_kind == 2 ? kind::POW_I : kind::POW;
  return b200_eltwise(e, &op, x, y, 0, 0, out, out_dims);
}

int32_t b200_scan(b200_engine* e, b200_buffer a, int32_t op, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "scan");
  if (st) return st;
  if (op < B200_SCAN_SUM || op > B200_SCAN_IMAX) return e->fail(B200_UNSUPPORTED, "scan: op %d", op);
  const int want = op >= B200_SCAN_ISUM ? B200_I32 : B200_F32;     // crates/tt-kernels/src/sfpu/scan.rs:44-49
  if (A->elem != want) return e->fail(B200_UNSUPPORTED, "scan: op %d takes elem %d, the buffer holds %d", op, want, A->elem);
  const uint64_t rows = A->rows, cols = A->cols;
  const uint32_t* src = (const uint32_t*)A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(rows, cols, want, out, &O);
  if (st) return st;
  uint32_t* dst = (uint32_t*)O->ptr;
  const uint64_t chunks = scan_chunks(op, rows, cols);
  void* carry = nullptr; uint64_t got = 0;
  if (chunks > 1) {
    st = e->alloc(chunks * cols * 4, &carry, &got);
    if (st) { e->drop(*out); return st; }
  }
  st = e->launched(launch_scan(src, dst, rows, cols, op, (uint32_t*)carry, e->stream), "scan", chunks > 1 ? 2 : 1);
  if (carry) e->release(carry, got);
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_sort_planes(b200_engine* e, b200_buffer a, int32_t elem, uint64_t n, int32_t descending, b200_buffer* keys,
                         b200_buffer* indices, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "sort_planes");
  if (st) return st;
  // crates/tt-kernels/src/sfpu/sort.rs:132-146 (what a sort refuses) and :705-713 (the planes' shape)
  if (elem != B200_F32 && elem != B200_I32) return e->fail(B200_UNSUPPORTED, "sort of elem %d (F32 and I32 only)", elem);
  if (n == 0) return e->fail(B200_UNSUPPORTED, "sort of an empty axis");
  if (n > 1024) return e->fail(B200_UNSUPPORTED, "axis length %llu exceeds the device sort's limit of 1024", (unsigned long long)n);
  if (A->elem != elem) return e->fail(B200_UNSUPPORTED, "sort_planes: the planes hold elem %d, the sort is of %d", A->elem, elem);
  uint64_t tiles = 1;
  while (tiles * 32 < n) tiles <<= 1;
  if (A->rows != 32 * tiles || A->cols % 32 != 0 || A->cols == 0)
    return e->fail(B200_UNSUPPORTED, "sort planes [%llu, %llu] for %llu axis positions (want [%llu, a multiple of 32])", (unsigned long long)A->rows,
                   (unsigned long long)A->cols, (unsigned long long)n, (unsigned long long)(32 * tiles));
  const uint64_t rows = A->rows, cols = A->cols;
  const uint32_t* src = (const uint32_t*)A->ptr;
  Buf *K = nullptr, *I = nullptr;
  st = e->new_buffer(rows, cols, elem, keys, &K);
  if (st) return st;
  uint32_t* kp = (uint32_t*)K->ptr;
  uint32_t* ip = nullptr;
  if (indices) {
    st = e->new_buffer(rows, cols, B200_I32, indices, &I);
    if (st) { e->drop(*keys); return st; }
    ip = (uint32_t*)I->ptr;
  }
  st = e->launched(launch_sort_planes(src, rows, cols, (uint32_t)n, elem == B200_I32, descending != 0, kp, ip, e->stream), "sort_planes");
  if (st) { e->drop(*keys); if (indices) e->drop(*indices); return st; }
  set_dims(out_dims, rows, cols);
  return B200_OK;
}

int32_t b200_random(b200_engine* e, const uint64_t dims[2], int32_t draw, float a, float b, int32_t lo, int32_t hi, int32_t as_int,
                    uint64_t base, b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  float p0 = a, p1 = b;
  int32_t i0 = 0, i1 = 0;
  int elem = B200_F32;
  switch (draw) {      // what each draw refuses: crates/tt-kernels/src/prng.rs:462-466, 487-491, 517-521, 574-578
    case 0: break;
    case 1: {
      const float scale = b - a;
      if (!(std::isfinite(a) && std::isfinite(b) && a < b && std::isfinite(scale) && scale > 0.0f))
        return e->fail(B200_UNSUPPORTED, "uniform [%g, %g) is not a finite, nonempty interval", a, b);
      uint32_t bits; memcpy(&bits, &b, 4);                  // the float below hi (prng.rs:322-329)
      if (b == 0.0f) bits = 0x80000001u; else bits = b > 0.0f ? bits - 1 : bits + 1;
      i1 = (int32_t)bits;
      break;
    }
    case 2:
      if (!(a >= 0.0f && a <= 1.0f)) return e->fail(B200_UNSUPPORTED, "Bernoulli probability %g is not in [0, 1]", a);
      if (as_int) elem = B200_I32;
      break;
    case 3:
      if (!(std::isfinite(a) && std::isfinite(b) && b >= 0.0f)) return e->fail(B200_UNSUPPORTED, "normal(mean %g, std %g) needs finite mean and std >= 0", a, b);
      if (as_int) elem = B200_I32;
      break;
    case 4: {
      const int64_t range = (int64_t)hi - (int64_t)lo;
      if (range < 1 || range > (1ll << 23))
        return e->fail(B200_UNSUPPORTED, "integer uniform [%d, %d): a range of %lld outside 1..=8388608", lo, hi, (long long)range);
      p0 = (float)range; i0 = lo; elem = B200_I32;
      break;
    }
    case 5: elem = B200_I32; break;
    default: return e->fail(B200_UNSUPPORTED, "random: draw %d", draw);
  }
  Buf* O = nullptr;
  int st = e->new_buffer(dims[0], dims[1], elem, out, &O);
  if (st) return st;
  st = e->launched(launch_random((uint32_t*)O->ptr, dims[0] * dims[1], draw, p0, p1, i0, i1, as_int != 0, base, e->stream), "random");
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, dims[0], dims[1]);
  return B200_OK;
}

int32_t b200_pool_bf16(b200_engine* e, b200_buffer a, const uint64_t* offsets, const uint64_t* coords, const uint64_t* divisors,
                       uint64_t n_windows, const uint64_t dims[2], b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf* A = nullptr;
  int st = e->need(a, &A, "pool_bf16");
  if (st) return st;
  if (A->elem != B200_BF16) return e->fail(B200_UNSUPPORTED, "pool_bf16: no BF16 buffer %llu", (unsigned long long)a);
  if (n_windows == 0 || dims[0] * dims[1] != n_windows) return e->fail(B200_UNSUPPORTED, "pool_bf16: invalid BF16 pool windows (%llu for [%llu, %llu])",
                                                                       (unsigned long long)n_windows, (unsigned long long)dims[0], (unsigned long long)dims[1]);
  const uint64_t total = offsets[n_windows];
  if (total > 0xffffffffull || A->rows * A->cols > 0xffffffffull) return e->fail(B200_UNSUPPORTED, "pool_bf16: more than 2^32 taps or elements");
  std::vector<uint32_t> meta(n_windows + 1 + total);      // offsets, then the taps' element offsets
  std::vector<float> div(n_windows);
  for (uint64_t w = 0; w < n_windows; ++w) {
    if (offsets[w + 1] <= offsets[w]) return e->fail(B200_UNSUPPORTED, "pool_bf16: window %llu is empty", (unsigned long long)w);
    if (divisors[w] == 0 || divisors[w] > (1ull << 24)) return e->fail(B200_UNSUPPORTED, "pool_bf16: divisor %llu of window %llu", (unsigned long long)divisors[w], (unsigned long long)w);
    meta[w] = (uint32_t)offsets[w];
    div[w] = (float)divisors[w];
  }
  meta[n_windows] = (uint32_t)total;
  for (uint64_t i = 0; i < total; ++i) {
    const uint64_t r = coords[2 * i], c = coords[2 * i + 1];
    if (r >= A->rows || c >= A->cols) return e->fail(B200_DOMAIN, "pool_bf16: DOMAIN: tap %llu names [%llu, %llu]", (unsigned long long)i, (unsigned long long)r, (unsigned long long)c);
    meta[n_windows + 1 + i] = (uint32_t)(r * A->cols + c);
  }
  const uint16_t* src = (const uint16_t*)A->ptr;
  Buf* O = nullptr;
  st = e->new_buffer(dims[0], dims[1], B200_F32, out, &O);
  if (st) return st;
  float* op = (float*)O->ptr;
  void *dm = nullptr, *dd = nullptr; uint64_t gm = 0, gd = 0;
  st = e->to_device(meta.data(), meta.size() * 4, &dm, &gm);
  if (!st) { st = e->to_device(div.data(), div.size() * 4, &dd, &gd); if (st) e->release(dm, gm); }
  if (st) { e->drop(*out); return st; }
  st = e->launched(launch_pool_windows(src, (const uint32_t*)dm, (const uint32_t*)dm + n_windows + 1, (const float*)dd, n_windows, op, e->stream), "pool_bf16");
  e->release(dm, gm); e->release(dd, gd);
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, dims[0], dims[1]);
  return B200_OK;
}

int32_t b200_metadata(b200_engine* e, const uint32_t* bits, const uint64_t dims[2], int32_t elem, b200_buffer* out) {
  if (elem != B200_F32 && elem != B200_I32 && elem != B200_BOOL)
    return e->fail(B200_UNSUPPORTED, "metadata: elem %d is not a 32-bit element", elem);
  if (!e->capturing) return upload_any(e, bits, dims[0], dims[1], elem, out);
  // Inside a capture the words become a copy node from memory the trace owns: every replay writes them again.
  cudaSetDevice(e->device);
  Buf* O = nullptr;
  int st = e->new_buffer(dims[0], dims[1], elem, out, &O);
  if (st) return st;
  const uint64_t bytes = dims[0] * dims[1] * 4;
  if (bytes) {
    void* pin = nullptr;
    if (cudaMallocHost(&pin, bytes) != cudaSuccess) { cudaGetLastError(); e->drop(*out); return e->fail(B200_OUT_OF_MEMORY, "trace: no pinned memory for metadata"); }
    memcpy(pin, bits, bytes);
    e->cur.pinned.push_back(pin);
    cudaError_t ce = cudaMemcpyAsync(O->ptr, pin, bytes, cudaMemcpyHostToDevice, e->stream);
    if (ce != cudaSuccess) { e->drop(*out); return e->cuda_fail(ce, "metadata"); }
    e->traffic.bytes_h2d += bytes;
  }
  return B200_OK;
}

int32_t b200_free_bytes(b200_engine* e, uint64_t out[2]) {
  cudaSetDevice(e->device);
  size_t fr = 0, tot = 0;
  cudaError_t ce = cudaMemGetInfo(&fr, &tot);
  if (ce != cudaSuccess) return e->cuda_fail(ce, "free_bytes");
  uint64_t idle = 0;
  for (auto& kv : e->cache) idle += kv.first;
  uint64_t driver = fr;
  if (e->cfg.pool_limit_bytes) {
    const uint64_t room = e->cfg.pool_limit_bytes > e->traffic.pool_reserved ? e->cfg.pool_limit_bytes - e->traffic.pool_reserved : 0;
    driver = std::min<uint64_t>(driver, room);
  }
  out[0] = driver + idle;   // idle blocks go back to the driver when a request does not fit them
  out[1] = driver + idle;
  return B200_OK;
}

// ---- one decode step through every layer, as one launch ---------------------------
// What a generation step (crates/tt-models/src/generate.rs:781) asks of the engine between the embedding and the head,
// as one cooperative kernel instead of eleven launches a layer (csrc/k_decode.cu).  An extension beside the trait, as
// `b200_attention_blocks` is: the composed step stays available and the two are held together by a test.
int32_t b200_decode_layers(b200_engine* e, const b200_decode_shape* shape, b200_buffer x, const b200_buffer* layer_buffers,
                           b200_buffer final_norm, b200_buffer cos_table, b200_buffer sin_table, b200_buffer position,
                           b200_buffer* out, uint64_t out_dims[2]) {
  cudaSetDevice(e->device);
  Buf *X = nullptr, *FN = nullptr, *CS = nullptr, *SN = nullptr, *P = nullptr;
  int st = e->need(x, &X, "decode_layers");
  if (!st) st = e->need(final_norm, &FN, "decode_layers");
  if (!st) st = e->need(cos_table, &CS, "decode_layers");
  if (!st) st = e->need(sin_table, &SN, "decode_layers");
  if (!st) st = e->need(position, &P, "decode_layers");
  if (st) return st;
  DecodeShape sh{};
  sh.layers = shape->layers; sh.rows = (uint32_t)X->rows; sh.hidden = shape->hidden; sh.heads = shape->heads;
  sh.kv_heads = shape->kv_heads; sh.head_dim = shape->head_dim; sh.ff = shape->ff; sh.max_len = shape->max_len;
  sh.attend = shape->attend; sh.eps = shape->eps; sh.scale = shape->scale;
  const char* why = "";
  if (X->rows > 4 || !decode_layers_supported(sh, &why))
    return e->fail(B200_UNSUPPORTED, "decode_layers: this kernel takes %s", X->rows > 4 ? "one to four sequences a step" : why);
  const uint64_t H = sh.hidden, QC = (uint64_t)sh.heads * 64, KC = (uint64_t)sh.kv_heads * 64, FF = sh.ff;
  if (X->elem != B200_F32 || X->cols != H) return e->fail(B200_UNSUPPORTED, "decode_layers: x must be F32 [rows, %llu]", (unsigned long long)H);
  if (FN->elem != B200_BF16 || FN->rows * FN->cols != H) return e->fail(B200_UNSUPPORTED, "decode_layers: the final gain must be BF16 of %llu values", (unsigned long long)H);
  if (CS->elem != B200_F32 || SN->elem != B200_F32 || CS->cols != 64 || SN->cols != 64 || CS->rows < sh.max_len || SN->rows < sh.max_len)
    return e->fail(B200_UNSUPPORTED, "decode_layers: the RoPE tables must be F32 [max_len, 64]");
  if (P->elem != B200_I32 || P->rows * P->cols != 1) return e->fail(B200_UNSUPPORTED, "decode_layers: the position must be one I32");
  std::vector<DecodeLayerPtrs> recs(sh.layers);
  for (uint32_t l = 0; l < sh.layers; ++l) {
    Buf* b[8];
    for (int i = 0; i < 8; ++i) {
      st = e->need(layer_buffers[(size_t)l * 8 + i], &b[i], "decode_layers", true);
      if (st) return st;
    }
    const uint64_t want[6][2] = {{1, H}, {H, QC + 2 * KC}, {QC, H}, {1, H}, {H, 2 * FF}, {FF, H}};
    for (int i = 0; i < 6; ++i) {
      const bool gain = i == 0 || i == 3;
      const bool shape_ok = gain ? b[i]->rows * b[i]->cols == H : (b[i]->rows == want[i][0] && b[i]->cols == want[i][1]);
      const bool elem_ok = gain ? b[i]->elem == B200_BF16 : (b[i]->elem == B200_BF16 || b[i]->elem == B200_BFP8);
      if (!shape_ok || !elem_ok)
        return e->fail(B200_UNSUPPORTED, "decode_layers: layer %u operand %d is [%llu,%llu] elem %d, not [%llu,%llu] %s", l, i,
                       (unsigned long long)b[i]->rows, (unsigned long long)b[i]->cols, b[i]->elem, (unsigned long long)want[i][0],
                       (unsigned long long)want[i][1], gain ? "BF16" : "BF16 or BFP8");
    }
    for (int i = 6; i < 8; ++i)
      if (b[i]->elem != B200_BF16 || b[i]->cols != KC || b[i]->rows != (uint64_t)sh.rows * sh.max_len)
        return e->fail(B200_UNSUPPORTED, "decode_layers: layer %u's cache must be BF16 [%llu, %llu]", l,
                       (unsigned long long)sh.rows * sh.max_len, (unsigned long long)KC);
    DecodeLayerPtrs& r = recs[l];
    r.norm1 = b[0]->ptr; r.qkv = b[1]->ptr; r.o = b[2]->ptr; r.norm2 = b[3]->ptr; r.gate_up = b[4]->ptr; r.down = b[5]->ptr;
    r.kc = b[6]->ptr; r.vc = b[7]->ptr;
    r.bfp = (b[1]->elem == B200_BFP8 ? 1u : 0u) | (b[2]->elem == B200_BFP8 ? 2u : 0u) | (b[4]->elem == B200_BFP8 ? 4u : 0u) |
            (b[5]->elem == B200_BFP8 ? 8u : 0u);
    r.pad = 0;
  }
  {
    bool any = false, all = true;
    for (const DecodeLayerPtrs& r : recs) { any = any || r.bfp != 0; all = all && r.bfp == 15u; }
    sh.weights = !any ? 0u : (all ? 1u : 2u);
  }
  const int grid = decode_layers_grid();
  const DecodeScratch cut = decode_layers_scratch(sh, grid);
  Buf* O = nullptr;
  st = e->new_buffer(sh.rows, H, B200_BF16, out, &O);
  if (st) return st;
  void *recs_dev = nullptr, *scratch = nullptr, *maps_dev = nullptr;
  uint64_t got_r = 0, got_s = 0, got_m = 0;
  st = e->to_device(recs.data(), recs.size() * sizeof(DecodeLayerPtrs), &recs_dev, &got_r);
  bool any_bfp = false;
  for (const DecodeLayerPtrs& r : recs) any_bfp = any_bfp || r.bfp != 0;
  if (!st && decode_layers_cluster_wanted(sh, any_bfp)) {   // the cluster form's descriptors; without an encoder the grid form runs
    std::vector<uint64_t> maps((decode_layers_maps_bytes(sh) + 7) / 8 + 8);
    void* aligned = reinterpret_cast<void*>(((uintptr_t)maps.data() + 63) & ~(uintptr_t)63);
    if (decode_layers_make_maps(sh, recs.data(), aligned)) st = e->to_device(aligned, decode_layers_maps_bytes(sh), &maps_dev, &got_m);
  }
  if (!st) st = e->alloc(cut.floats * sizeof(float), &scratch, &got_s);
  if (!st) {
    X = e->get(x); FN = e->get(final_norm); CS = e->get(cos_table); SN = e->get(sin_table); P = e->get(position); O = e->get(*out);
    st = e->launched(launch_decode_layers(sh, (const DecodeLayerPtrs*)recs_dev, (const float*)X->ptr, FN->ptr, (const float*)CS->ptr,
                                          (const float*)SN->ptr, (const int32_t*)P->ptr, (uint16_t*)O->ptr, (float*)scratch, cut, grid,
                                          maps_dev, e->d_err, e->stream, &e->decode_form), "decode_layers");
  }
  if (scratch) e->release(scratch, got_s);
  if (recs_dev) e->release(recs_dev, got_r);
  if (maps_dev) e->release(maps_dev, got_m);
  if (st) { e->drop(*out); return st; }
  set_dims(out_dims, sh.rows, H);
  return B200_OK;
}

// ---- traces: server.rs:591-660 ---------------------------------------------------
int32_t b200_begin_trace(b200_engine* e) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "begin_trace: a capture is already open");
  int st = e->wait();  // nothing pending, no earlier failure
  if (st) return st;
  cudaError_t ce = cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed);
  if (ce != cudaSuccess) return e->cuda_fail(ce, "begin_trace");
  e->capturing = true;
  e->cur = b200_engine::Trace();
  e->cur_free.clear();
  e->cur_owned.clear();
  return B200_OK;
}

int32_t b200_end_trace(b200_engine* e, uint64_t* trace) {
  cudaSetDevice(e->device);
  if (!e->capturing) return e->fail(B200_UNSUPPORTED, "end_trace: no capture is open");
  e->capturing = false;
  cudaGraph_t g = nullptr;
  cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
  if (ce == cudaSuccess) { e->cur.graph = g; ce = cudaGraphInstantiate(&e->cur.exec, g, 0); }
  if (ce != cudaSuccess) {
    cudaGetLastError();
    if (g) cudaGraphDestroy(g);
    for (void* h : e->cur.pinned) cudaFreeHost(h);
    // the blocks go back to the pool; buffers made during the failed capture stay valid
    for (auto& kv : e->cur_free) e->cache.emplace(kv.first, kv.second);
    e->cur_free.clear(); e->cur_owned.clear();
    return e->cuda_fail(ce, "end_trace");
  }
  e->cur_free.clear();
  e->cur_owned.clear();
  *trace = e->next_trace++;
  for (auto& b : e->cur.blocks) e->trace_ptrs.insert(b.first);
  e->traces.emplace(*trace, std::move(e->cur));
  e->cur = b200_engine::Trace();
  return B200_OK;
}

int32_t b200_run_trace(b200_engine* e, uint64_t trace) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "run_trace inside a capture");
  auto it = e->traces.find(trace);
  if (it == e->traces.end()) return e->fail(B200_STALE, "run_trace: no trace %llu", (unsigned long long)trace);
  cudaError_t ce = cudaGraphLaunch(it->second.exec, e->stream);
  if (ce != cudaSuccess) return e->cuda_fail(ce, "run_trace");
  e->traffic.launches += it->second.launches;
  return B200_OK;
}

void b200_release_trace(b200_engine* e, uint64_t trace) {
  cudaSetDevice(e->device);
  auto it = e->traces.find(trace);
  if (it == e->traces.end()) return;
  cudaStreamSynchronize(e->stream);
  b200_engine::Trace t = std::move(it->second);
  e->traces.erase(it);
  if (t.exec) cudaGraphExecDestroy(t.exec);
  if (t.graph) cudaGraphDestroy(t.graph);
  for (void* h : t.pinned) cudaFreeHost(h);
  // Blocks no live buffer sits in return to the pool; the rest return when their buffer is freed.
  for (auto& b : t.blocks) e->trace_ptrs.erase(b.first);
  for (auto& b : t.blocks) {
    bool live = false;
    for (auto& kv : e->bufs) if (kv.second.ptr == b.first && !kv.second.parent) { live = true; break; }
    if (!live) e->cache.emplace(b.second, b.first);
  }
}

// ---- waits and observability ---------------------------------------------------
int32_t b200_sync(b200_engine* e) { cudaSetDevice(e->device); return e->wait(); }
void b200_set_op_label(b200_engine* e, const char* label) {
  e->label = label ? label : "";
  if (e->profiling && !e->capturing) {
    cudaSetDevice(e->device);
    b200_engine::Mark m;
    m.label = e->label;
    m.launches = e->traffic.launches;
    if (cudaEventCreate(&m.at) == cudaSuccess && cudaEventRecord(m.at, e->stream) == cudaSuccess) e->marks.push_back(m);
    else { if (m.at) cudaEventDestroy(m.at); cudaGetLastError(); }
  }
}

// ---- per-op device time: profile.rs:1-48, report.rs:27-55 -----------------------------
int32_t b200_profile_start(b200_engine* e) {
  cudaSetDevice(e->device);
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "profile_start inside a trace capture");
  e->drop_marks();
  e->prof_table.clear();
  e->profiling = true;
  return B200_OK;
}
int32_t b200_profile_stop(b200_engine* e) {
  cudaSetDevice(e->device);
  if (!e->profiling) return e->fail(B200_UNSUPPORTED, "profile_stop: the profile mode is off");
  if (e->capturing) return e->fail(B200_UNSUPPORTED, "profile_stop inside a trace capture");
  e->profiling = false;
  const uint64_t launches_end = e->traffic.launches;
  cudaError_t ce = cudaEventCreate(&e->prof_end);
  if (ce == cudaSuccess) ce = cudaEventRecord(e->prof_end, e->stream);
  if (ce != cudaSuccess) { e->drop_marks(); return e->cuda_fail(ce, "profile_stop"); }
  const int st = e->wait();
  if (st) { e->drop_marks(); return st; }
  for (size_t i = 0; i < e->marks.size(); ++i) {
    const bool last = i + 1 == e->marks.size();
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, e->marks[i].at, last ? e->prof_end : e->marks[i + 1].at) != cudaSuccess) { cudaGetLastError(); ms = 0.f; }
    const uint64_t l1 = last ? launches_end : e->marks[i + 1].launches;
    b200_engine::Stat* stat = nullptr;
    for (auto& kv : e->prof_table) if (kv.first == e->marks[i].label) { stat = &kv.second; break; }
    if (!stat) { e->prof_table.emplace_back(e->marks[i].label, b200_engine::Stat()); stat = &e->prof_table.back().second; }
    stat->calls += 1;
    stat->launches += l1 - e->marks[i].launches;
    stat->ms += (double)ms;
  }
  e->drop_marks();
  return B200_OK;
}
int32_t b200_profile_read(const b200_engine* e, b200_op_stat* out, uint64_t capacity, uint64_t* n) {
  if (n) *n = e->prof_table.size();
  for (uint64_t i = 0; out && i < capacity && i < e->prof_table.size(); ++i) {
    memset(&out[i], 0, sizeof out[i]);
    strncpy(out[i].op, e->prof_table[i].first.c_str(), sizeof out[i].op - 1);
    out[i].calls = e->prof_table[i].second.calls;
    out[i].launches = e->prof_table[i].second.launches;
    out[i].device_ms = e->prof_table[i].second.ms;
  }
  return B200_OK;
}

// server.rs:730 `trace_footprint`: the device bytes a trace holds until it is released.
int32_t b200_trace_footprint(const b200_engine* e, uint64_t trace, uint64_t* bytes) {
  auto it = e->traces.find(trace);
  if (it == e->traces.end()) return B200_STALE;
  uint64_t total = 0;
  for (auto& b : it->second.blocks) total += b.second;
  *bytes = total;
  return B200_OK;
}

// server.rs:664 `trace_ops`: the ops a trace captured, in capture order, each with the label it ran under
// and the kernels it launched (`device_ms` is 0: a replay is timed as a whole, under its own label).
int32_t b200_trace_ops(const b200_engine* e, uint64_t trace, b200_op_stat* out, uint64_t capacity, uint64_t* n) {
  auto it = e->traces.find(trace);
  if (it == e->traces.end()) return B200_STALE;
  const auto& ops = it->second.ops;
  if (n) *n = ops.size();
  for (uint64_t i = 0; out && i < capacity && i < ops.size(); ++i) {
    memset(&out[i], 0, sizeof out[i]);
    strncpy(out[i].op, ops[i].first.c_str(), sizeof out[i].op - 1);
    out[i].calls = 1;
    out[i].launches = ops[i].second;
  }
  return B200_OK;
}

// A bounded device wait that nothing ends, run on purpose: the one failure a kernel of this engine can meet
// on a healthy GPU.  The wait gives up at the engine's limit, the next wait reports TIMEOUT
// (crates/burn-tt/src/error.rs:40), the GPU and the CUDA context stay usable.
int32_t b200_debug_stalled_wait(b200_engine* e) {
  cudaSetDevice(e->device);
  if (e->wait_limit_word <= 0 || e->wait_limit_word > 2000000000ll)
    return e->fail(B200_UNSUPPORTED, "debug_stalled_wait: set b200_config.wait_limit_cycles to at most 2e9 (a second) first");
  return e->launched(launch_stalled_wait(e->d_err, e->stream), "debug_stalled_wait");
}
void b200_set_matmul_sm_limit(b200_engine* e, int32_t sms) { e->matmul_sm_limit = sms > 0 ? sms : 0; }
void b200_traffic_get(const b200_engine* e, b200_traffic* out) { *out = e->traffic; }
int32_t b200_timer_start(b200_engine* e) {
  cudaSetDevice(e->device);
  cudaError_t ce = cudaEventRecord(e->t0, e->stream);
  return ce == cudaSuccess ? B200_OK : e->cuda_fail(ce, "timer_start");
}
int32_t b200_timer_stop(b200_engine* e, float* ms) {
  cudaSetDevice(e->device);
  cudaError_t ce = cudaEventRecord(e->t1, e->stream);
  if (ce == cudaSuccess) ce = cudaEventSynchronize(e->t1);
  if (ce == cudaSuccess) ce = cudaEventElapsedTime(ms, e->t0, e->t1);
  return ce == cudaSuccess ? B200_OK : e->cuda_fail(ce, "timer_stop");
}
void* b200_stream(const b200_engine* e) { return (void*)e->stream; }
const char* b200_last_matmul_path(const b200_engine* e) { return e->matmul_path; }
const char* b200_last_decode_form(const b200_engine* e) { return e->decode_form; }

}  // extern "C"
