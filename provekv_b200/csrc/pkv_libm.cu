// Tables that let the kernels reproduce the host libm's logf / expf bit for bit.
//
// The reference computes BlockLogU8 radii with the platform libm through Rust std
// (turbo-quant/src/radius.rs:61 `ln`, :143 `exp`); glibc's binary32 functions are within one unit
// in the last place of the correctly rounded result but not always equal to it, so a wire written
// on one machine is defined by that machine's libm.  The kernels evaluate the correctly rounded
// functions of include/pkv_portable_math.h.  For a profile created with PKV_LIBM_PLATFORM the
// library scans every binary32 argument in the function's domain once per process on the host
// (about two seconds per function on 16 cores), keeps the arguments where the host function's
// bits differ from the portable one's (a few 1e-4 of them, all by one unit), and uploads them as
// a sorted key array with a direction bit per key and a Bloom-style bitmap in front of it.  A
// device lookup is one bitmap probe, and a binary search for the ~2 % of probes that hit.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <thread>
#include <vector>

#include "pkv_common.cuh"

namespace {

struct HostTable {
  std::vector<uint32_t> keys;  // argument bit patterns, ascending as unsigned integers
  std::vector<uint32_t> dirs;  // bit i: host bits = portable bits + 1 (else - 1)
  bool ok = false;             // every difference was exactly one unit
  bool built = false;
};

float host_fn(int kind, float x) { return kind == PKV_LIBM_FN_LOG ? logf(x) : expf(x); }
float portable_fn(int kind, float x) { return kind == PKV_LIBM_FN_LOG ? pkv_logf_portable(x) : pkv_expf_portable(x); }

// Argument ranges (inclusive bit patterns).  logf: positive normal numbers (radii are clamped to
// FLT_MIN, radius.rs:61).  expf: |t| <= 89 covers every min + span * q / 255 between the logs of
// FLT_MIN and FLT_MAX; both signs.
void domain(int kind, std::vector<std::pair<uint32_t, uint32_t>>* ranges) {
  if (kind == PKV_LIBM_FN_LOG) {
    ranges->push_back({0x00800000u, 0x7f7fffffu});
  } else {
    ranges->push_back({0x00000000u, 0x42b20000u});
    ranges->push_back({0x80000000u, 0xc2b20000u});
  }
}

void scan(int kind, uint32_t lo, uint32_t hi, std::vector<uint32_t>* keys, std::vector<uint8_t>* up, bool* ok) {
  for (uint64_t u64 = lo; u64 <= hi; u64++) {
    const uint32_t u = (uint32_t)u64;
    float x;
    memcpy(&x, &u, 4);
    const float h = host_fn(kind, x), p = portable_fn(kind, x);
    uint32_t hb, pb;
    memcpy(&hb, &h, 4);
    memcpy(&pb, &p, 4);
    if (hb == pb) continue;
    if (hb == pb + 1u) up->push_back(1);
    else if (hb + 1u == pb) up->push_back(0);
    else {
      *ok = false;
      up->push_back(0);
    }
    keys->push_back(u);
  }
}

HostTable* host_table(int kind) {
  static HostTable tables[2];
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  HostTable* t = &tables[kind];
  if (t->built) return t;
  std::vector<std::pair<uint32_t, uint32_t>> ranges;
  domain(kind, &ranges);
  unsigned nt = std::thread::hardware_concurrency();
  if (nt == 0) nt = 4;
  if (nt > 64) nt = 64;
  t->ok = true;
  for (const auto& r : ranges) {
    const uint64_t span = (uint64_t)r.second - r.first + 1;
    std::vector<std::vector<uint32_t>> keys(nt);
    std::vector<std::vector<uint8_t>> ups(nt);
    std::vector<char> oks(nt, 1);
    std::vector<std::thread> th;
    for (unsigned i = 0; i < nt; i++) {
      const uint32_t lo = r.first + (uint32_t)(span * i / nt);
      const uint32_t hi = r.first + (uint32_t)(span * (i + 1) / nt - 1);
      th.emplace_back([=, &keys, &ups, &oks]() {
        bool ok = true;
        scan(kind, lo, hi, &keys[i], &ups[i], &ok);
        oks[i] = ok;
      });
    }
    for (auto& x : th) x.join();
    for (unsigned i = 0; i < nt; i++) {
      if (!oks[i]) t->ok = false;
      for (size_t k = 0; k < keys[i].size(); k++) {
        const size_t idx = t->keys.size();
        if ((idx & 31) == 0) t->dirs.push_back(0);
        if (ups[i][k]) t->dirs.back() |= 1u << (idx & 31);
        t->keys.push_back(keys[i][k]);
      }
    }
  }
  t->built = true;
  return t;
}

struct DeviceTable {
  PkvUlpTable dev = {nullptr, nullptr, nullptr, 0, 0};
  bool ready = false;
};

}  // namespace

// The table of `kind` in the memory of the current device (built and uploaded on first use).
int pkv_ulp_table_get(int kind, PkvUlpTable* out) {
  static DeviceTable cache[2][64];
  static std::mutex mu;
  if (kind < 0 || kind > 1 || !out) return PKV_ERR_INVALID_ARGUMENT;
  int dev = 0;
  if (cudaError_t ce = cudaGetDevice(&dev)) return pkv_cuda_status(ce);
  if (dev < 0 || dev >= 64) return PKV_ERR_UNSUPPORTED;
  HostTable* h = host_table(kind);
  if (!h->ok) return PKV_ERR_UNSUPPORTED;  // a difference of more than one unit: not representable here
  std::lock_guard<std::mutex> lock(mu);
  DeviceTable* d = &cache[kind][dev];
  if (!d->ready) {
    const uint32_t n = (uint32_t)h->keys.size();
    uint32_t bits = 1u << 16;
    while (bits < 64u * n && bits < (1u << 30)) bits <<= 1;
    std::vector<uint32_t> bloom(bits / 32, 0u);
    for (uint32_t k : h->keys) {
      const uint32_t b = (k * PKV_ULP_HASH_MUL) >> (32 - __builtin_ctz(bits));
      bloom[b >> 5] |= 1u << (b & 31);
    }
    uint32_t *keys = nullptr, *dirs = nullptr, *bl = nullptr;
    cudaError_t e = cudaMalloc((void**)&keys, sizeof(uint32_t) * (n + 1));
    if (e == cudaSuccess) e = cudaMalloc((void**)&dirs, sizeof(uint32_t) * (h->dirs.size() + 1));
    if (e == cudaSuccess) e = cudaMalloc((void**)&bl, sizeof(uint32_t) * bloom.size());
    if (e == cudaSuccess && n) e = cudaMemcpy(keys, h->keys.data(), sizeof(uint32_t) * n, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && n)
      e = cudaMemcpy(dirs, h->dirs.data(), sizeof(uint32_t) * h->dirs.size(), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(bl, bloom.data(), sizeof(uint32_t) * bloom.size(), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      if (keys) cudaFree(keys);
      if (dirs) cudaFree(dirs);
      if (bl) cudaFree(bl);
      return pkv_cuda_status(e);
    }
    d->dev = PkvUlpTable{keys, dirs, bl, n, (uint32_t)__builtin_ctz(bits)};
    d->ready = true;
  }
  *out = d->dev;
  return PKV_OK;
}

extern "C" int pkv_host_libm_exceptions(int32_t function, uint32_t* keys_out, int64_t capacity, int64_t* count,
                                        int32_t* all_one_unit) {
  if ((function != PKV_LIBM_FN_LOG && function != PKV_LIBM_FN_EXP) || !count) return PKV_ERR_INVALID_ARGUMENT;
  HostTable* h = host_table(function);
  *count = (int64_t)h->keys.size();
  if (all_one_unit) *all_one_unit = h->ok ? 1 : 0;
  if (keys_out)
    for (int64_t i = 0; i < capacity && i < *count; i++) keys_out[i] = h->keys[(size_t)i];
  return PKV_OK;
}
