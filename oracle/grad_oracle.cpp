// CPU oracle for the dense-contraction path of hyunjun3952/grad.  TEST INFRASTRUCTURE ONLY:
// the checker for the CUDA kernels and the timed CPU baseline; the product never links it.
// Parity status: pinned by the reference's own known-answer and exact-equality tests, which
// tests/test_oracle_golden.py replays against this file.  Each function cites the reference
// file:line whose arithmetic (operation order, rounding points, chunking) it restates.
#include "grad_oracle.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

namespace {

// ---------------------------------------------------------------------------------------------
// Worker pool.  The reference keeps up to 15 parked workers fed through mailboxes
// (src/cpu/kernels.zig:100-171); part 0 runs on the caller.  Only the partitioning affects results,
// so this pool is a plain mutex/condvar one with the same part numbering.
// ---------------------------------------------------------------------------------------------
constexpr size_t kMaxWorkers = 15;            // src/cpu/kernels.zig:101
constexpr size_t kMinFlopsPerPart = 2000000;  // src/cpu/kernels.zig:100

class Pool {
 public:
  static Pool& get() {
    static Pool* pool = new Pool();   // leaked on purpose: workers are detached
    return *pool;
  }
  // Runs fn(part) for part in [0, parts): part 0 on the caller, the rest on workers (the caller
  // helps with whatever is still unclaimed once its own part is done).
  void run(size_t parts, const std::function<void(size_t)>& fn) {
    if (parts <= 1) {
      fn(0);
      return;
    }
    std::lock_guard<std::mutex> serial(entry_);   // one job at a time, like the reference's single pool
    {
      std::unique_lock<std::mutex> lock(mu_);
      while (workers_ < std::min(parts - 1, kMaxWorkers)) {
        std::thread([this] { loop(); }).detach();
        ++workers_;
      }
      fn_ = &fn;
      parts_ = parts;
      next_ = 1;
      pending_ = parts - 1;
    }
    wake_.notify_all();
    fn(0);
    std::unique_lock<std::mutex> lock(mu_);
    while (next_ < parts_) {
      const size_t part = next_++;
      lock.unlock();
      fn(part);
      lock.lock();
      --pending_;
    }
    done_.wait(lock, [this] { return pending_ == 0; });
    fn_ = nullptr;
  }

 private:
  void loop() {
    std::unique_lock<std::mutex> lock(mu_);
    for (;;) {
      wake_.wait(lock, [this] { return fn_ != nullptr && next_ < parts_; });
      const size_t part = next_++;
      const std::function<void(size_t)>* fn = fn_;
      lock.unlock();
      (*fn)(part);
      lock.lock();
      if (--pending_ == 0) done_.notify_all();
    }
  }
  std::mutex entry_, mu_;
  std::condition_variable wake_, done_;
  const std::function<void(size_t)>* fn_ = nullptr;
  size_t workers_ = 0, parts_ = 0, pending_ = 0, next_ = 0;
};

// src/cpu/kernels.zig:203-218 `parallelFor`: parts = min(threads, 16, len / min_chunk), equal chunks.
template <class Body>
void parallel_for(int threads, size_t len, size_t min_chunk, const Body& body) {
  size_t parts = 1;
  if (threads > 1) parts = std::max<size_t>(1, std::min<size_t>({(size_t)threads, kMaxWorkers + 1, len / min_chunk}));
  if (parts == 1) {
    body(0, len);
    return;
  }
  const size_t chunk = (len + parts - 1) / parts;
  Pool::get().run(parts, [&](size_t p) {
    const size_t lo = std::min(p * chunk, len);
    body(lo, std::min(lo + chunk, len));
  });
}

int simd_lanes() {
#if defined(__x86_64__)
  static const int lanes = [] {
    if (std::getenv("GRAD_ORACLE_SCALAR")) return 0;
    if (__builtin_cpu_supports("avx512f")) return 16;
    if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 8;
    return 0;
  }();
  return lanes;
#else
  return 0;
#endif
}

// Lanes the reference would report through std.simd.suggestVectorLength(f32) on this host.  It only
// shapes the packing and two dispatch conditions (c_out % lanes), never the order of operations
// within one output element.
size_t lane_count_f32() { return simd_lanes() == 16 ? 16 : 8; }
template <class T> size_t lane_count();
template <> size_t lane_count<float>() { return lane_count_f32(); }
template <> size_t lane_count<double>() { return lane_count_f32() / 2; }

size_t round_up(size_t x, size_t to) { return (x + to - 1) / to * to; }

struct TileConfig {
  size_t mr = 6, nv = 2, mc = 96, kc = 256, nc = 1024;   // src/cpu/kernels.zig:61-70
  bool trans_a = false, trans_b = false, accumulate = false;
};

struct Split {
  int axis;   // 0 rows, 1 cols, 2 depth
  size_t parts, chunk;
};

// src/cpu/kernels.zig:234-249 `splitFor`.
template <class T>
Split split_for(const TileConfig& cfg, int threads, size_t m, size_t k, size_t n) {
  const bool by_rows = m >= n;
  const size_t unit = by_rows ? cfg.mr : cfg.nv * lane_count<T>();
  const size_t tiles = ((by_rows ? m : n) + unit - 1) / unit;
  const size_t by_work = 2 * m * k * n / kMinFlopsPerPart;
  const size_t want = threads <= 1 ? 1 : std::max<size_t>(1, std::min<size_t>({(size_t)threads, kMaxWorkers + 1, by_work}));
  if (tiles < want && k >= want * cfg.kc) {
    const size_t per = round_up((k + want - 1) / want, cfg.kc);
    return {2, (k + per - 1) / per, per};
  }
  const size_t per = (tiles + want - 1) / want;
  return {by_rows ? 0 : 1, (tiles + per - 1) / per, per * unit};
}

template <class T>
struct Problem {
  size_t m, k, n;
  const T* a;
  const T* b;
  T* out;
};

struct Range {
  size_t r0, r1, c0, c1, k0, k1;
};

// src/cpu/kernels.zig:265-295 `packB`: strips of NR columns, kc rows each, zero-padded columns.
template <class T>
void pack_b(size_t NR, bool trans, const Problem<T>& p, size_t pc, size_t jc, size_t kc, size_t nc, T* dst) {
  for (size_t jr = 0; jr < nc; jr += NR) {
    T* strip = dst + (jr / NR) * kc * NR;
    const size_t cols = std::min(NR, nc - jr);
    if (trans) {
      for (size_t c = 0; c < NR; ++c) {
        if (c < cols) {
          const T* src = p.b + (jc + jr + c) * p.k + pc;
          for (size_t q = 0; q < kc; ++q) strip[q * NR + c] = src[q];
        } else {
          for (size_t q = 0; q < kc; ++q) strip[q * NR + c] = 0;
        }
      }
    } else {
      for (size_t q = 0; q < kc; ++q) {
        const T* src = p.b + (pc + q) * p.n + jc + jr;
        T* row = strip + q * NR;
        for (size_t c = 0; c < cols; ++c) row[c] = src[c];
        for (size_t c = cols; c < NR; ++c) row[c] = 0;
      }
    }
  }
}

// src/cpu/kernels.zig:297-326 `microTile`: acc[r][c] = fma(a[r][p], b[p][c], acc[r][c]) for p ascending.
// One fused multiply-add per (r, c, p); the lane width changes nothing within an element.
template <class T>
void micro_tile_scalar(size_t MR, size_t NR, size_t kc, const T* a, const size_t* a_off, size_t a_step, const T* bp, T* acc) {
  for (size_t i = 0; i < MR * NR; ++i) acc[i] = 0;
  for (size_t p = 0; p < kc; ++p) {
    const T* brow = bp + p * NR;
    for (size_t r = 0; r < MR; ++r) {
      const T av = a[a_off[r] + p * a_step];
      T* arow = acc + r * NR;
      for (size_t c = 0; c < NR; ++c) arow[c] = std::fma(av, brow[c], arow[c]);
    }
  }
}

#if defined(__x86_64__)
__attribute__((target("avx2,fma"))) void micro_tile_6x16(size_t kc, const float* a, const size_t* a_off, size_t a_step,
                                                         const float* bp, float* acc) {
  __m256 c[6][2];
  for (int r = 0; r < 6; ++r) c[r][0] = c[r][1] = _mm256_setzero_ps();
  for (size_t p = 0; p < kc; ++p) {
    const __m256 b0 = _mm256_loadu_ps(bp + p * 16);
    const __m256 b1 = _mm256_loadu_ps(bp + p * 16 + 8);
    for (int r = 0; r < 6; ++r) {
      const __m256 av = _mm256_broadcast_ss(a + a_off[r] + p * a_step);
      c[r][0] = _mm256_fmadd_ps(av, b0, c[r][0]);
      c[r][1] = _mm256_fmadd_ps(av, b1, c[r][1]);
    }
  }
  for (int r = 0; r < 6; ++r) {
    _mm256_storeu_ps(acc + r * 16, c[r][0]);
    _mm256_storeu_ps(acc + r * 16 + 8, c[r][1]);
  }
}

__attribute__((target("avx512f"))) void micro_tile_6x32(size_t kc, const float* a, const size_t* a_off, size_t a_step,
                                                        const float* bp, float* acc) {
  __m512 c[6][2];
  for (int r = 0; r < 6; ++r) c[r][0] = c[r][1] = _mm512_setzero_ps();
  for (size_t p = 0; p < kc; ++p) {
    const __m512 b0 = _mm512_loadu_ps(bp + p * 32);
    const __m512 b1 = _mm512_loadu_ps(bp + p * 32 + 16);
    for (int r = 0; r < 6; ++r) {
      const __m512 av = _mm512_set1_ps(a[a_off[r] + p * a_step]);
      c[r][0] = _mm512_fmadd_ps(av, b0, c[r][0]);
      c[r][1] = _mm512_fmadd_ps(av, b1, c[r][1]);
    }
  }
  for (int r = 0; r < 6; ++r) {
    _mm512_storeu_ps(acc + r * 32, c[r][0]);
    _mm512_storeu_ps(acc + r * 32 + 16, c[r][1]);
  }
}
#endif

template <class T>
void micro_tile(size_t MR, size_t NR, size_t kc, const T* a, const size_t* a_off, size_t a_step, const T* bp, T* acc) {
  micro_tile_scalar<T>(MR, NR, kc, a, a_off, a_step, bp, acc);
}
template <>
void micro_tile<float>(size_t MR, size_t NR, size_t kc, const float* a, const size_t* a_off, size_t a_step, const float* bp, float* acc) {
#if defined(__x86_64__)
  if (MR == 6 && NR == 32 && simd_lanes() == 16) return micro_tile_6x32(kc, a, a_off, a_step, bp, acc);
  if (MR == 6 && NR == 16 && simd_lanes() == 8) return micro_tile_6x16(kc, a, a_off, a_step, bp, acc);
#endif
  micro_tile_scalar<float>(MR, NR, kc, a, a_off, a_step, bp, acc);
}

// src/cpu/kernels.zig:368-448 `matmulTiledRange`.  Per output element: start from 0 (or the old
// value when accumulating); for every KC-chunk of the depth range, in order, a fresh FMA chain over
// the chunk is added to the output with one rounding.
template <class T>
void matmul_tiled_range(const TileConfig& cfg, const Problem<T>& p, const Range& rg, T* work) {
  const size_t m = p.m, k = p.k, n = p.n;
  const size_t MR = cfg.mr, MC = cfg.mc, KC = cfg.kc, NC = cfg.nc;
  const size_t NR = cfg.nv * lane_count<T>();
  T* b_pack = work;
  if (!cfg.accumulate) {
    for (size_t r = rg.r0; r < rg.r1; ++r) std::fill(p.out + r * n + rg.c0, p.out + r * n + rg.c1, T(0));
  }
  std::vector<T> acc(MR * NR);
  std::vector<size_t> a_off(MR);
  for (size_t jc = rg.c0; jc < rg.c1; jc += NC) {
    const size_t nc = std::min(NC, rg.c1 - jc);
    for (size_t pc = rg.k0; pc < rg.k1; pc += KC) {
      const size_t kc = std::min(KC, rg.k1 - pc);
      pack_b<T>(NR, cfg.trans_b, p, pc, jc, kc, nc, b_pack);
      for (size_t ic = rg.r0; ic < rg.r1; ic += MC) {
        const size_t mc = std::min(MC, rg.r1 - ic);
        for (size_t jr = 0; jr < nc; jr += NR) {
          const size_t nr_eff = std::min(NR, nc - jr);
          const T* bp = b_pack + (jr / NR) * kc * NR;
          for (size_t ir = 0; ir < mc; ir += MR) {
            const size_t mr_eff = std::min(MR, mc - ir);
            for (size_t r = 0; r < MR; ++r) {
              const size_t row = ic + ir + std::min(r, mr_eff - 1);
              a_off[r] = cfg.trans_a ? pc * m + row : row * k + pc;
            }
            micro_tile<T>(MR, NR, kc, p.a, a_off.data(), cfg.trans_a ? m : 1, bp, acc.data());
            T* c = p.out + (ic + ir) * n + jc + jr;
            for (size_t r = 0; r < mr_eff; ++r)
              for (size_t cc = 0; cc < nr_eff; ++cc) c[r * n + cc] += acc[r * NR + cc];
          }
        }
      }
    }
  }
}

template <class T>
size_t part_work_len(const TileConfig& cfg, const Split& s, size_t m, size_t k, size_t n) {
  const size_t ncols = s.axis == 1 ? std::min(n, s.chunk) : n;
  const size_t kc = std::min(cfg.kc, k);
  const size_t nc = std::min(cfg.nc, round_up(ncols, cfg.nv * lane_count<T>()));
  return kc * nc + (s.axis == 2 ? m * n : 0);
}

// src/cpu/kernels.zig:328-365 `matmulTiled`: a depth split gives later parts a private zeroed output
// which is added to the real output in part order after all parts finish.
template <class T>
void matmul_tiled(const TileConfig& cfg, int threads, const Problem<T>& p) {
  if (p.m == 0 || p.n == 0) return;
  const Split s = split_for<T>(cfg, threads, p.m, p.k, p.n);
  const size_t part_len = part_work_len<T>(cfg, s, p.m, p.k, p.n);
  std::vector<T> work(s.parts * part_len);
  const Range whole{0, p.m, 0, p.n, 0, p.k};
  if (s.parts == 1) {
    matmul_tiled_range<T>(cfg, p, whole, work.data());
    return;
  }
  Pool::get().run(s.parts, [&](size_t part) {
    const size_t lo = part * s.chunk;
    T* w = work.data() + part * part_len;
    Range rg = whole;
    if (s.axis == 0) { rg.r0 = lo; rg.r1 = std::min(lo + s.chunk, p.m); }
    if (s.axis == 1) { rg.c0 = lo; rg.c1 = std::min(lo + s.chunk, p.n); }
    if (s.axis == 2) { rg.k0 = lo; rg.k1 = std::min(lo + s.chunk, p.k); }
    if (s.axis != 2 || part == 0) {
      matmul_tiled_range<T>(cfg, p, rg, w);
      return;
    }
    TileConfig fresh = cfg;
    fresh.accumulate = false;
    Problem<T> own = p;
    own.out = w + part_len - p.m * p.n;
    matmul_tiled_range<T>(fresh, own, rg, w);
  });
  if (s.axis == 2) {
    for (size_t part = 1; part < s.parts; ++part) {
      const T* own = work.data() + (part + 1) * part_len - p.m * p.n;
      for (size_t i = 0; i < p.m * p.n; ++i) p.out[i] += own[i];
    }
  }
}

template <class T>
void matmul_naive(size_t m, size_t k, size_t n, const T* a, const T* b, T* out) {
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      volatile T acc = 0;   // volatile keeps the separate multiply and add (no contraction to FMA)
      for (size_t q = 0; q < k; ++q) {
        const T prod = a[i * k + q] * b[q * n + j];
        acc = acc + prod;
      }
      out[i * n + j] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// Convolution geometry, src/gpu/math/conv.zig:22-65.
// ---------------------------------------------------------------------------------------------
using Dims = oracle_dims;
uint32_t out_h(const Dims& d) { return (d.h + 2 * d.pad - d.dilation * (d.k - 1) - 1) / d.stride + 1; }
uint32_t out_w(const Dims& d) { return (d.w + 2 * d.pad - d.dilation * (d.k - 1) - 1) / d.stride + 1; }
size_t rows_of(const Dims& d) { return (size_t)d.n * out_h(d) * out_w(d); }
size_t patch_len(const Dims& d) { return (size_t)d.k * d.k * d.c; }

struct Patch {
  uint32_t n, top, left;
};
Patch patch_of(uint32_t row, const Dims& d) {
  const uint32_t ow = out_w(d), oh = out_h(d);
  return {row / ow / oh, row / ow % oh * d.stride, row % ow * d.stride};
}
// src/gpu/math/conv.zig:58-65 `patchSource`; -1 stands for the padding.
int64_t patch_source(const Patch& pt, uint32_t cc, const Dims& d) {
  const uint32_t tap = cc / d.c;
  const uint32_t py = pt.top + tap / d.k * d.dilation;
  const uint32_t px = pt.left + tap % d.k * d.dilation;
  if (py < d.pad || px < d.pad || py - d.pad >= d.h || px - d.pad >= d.w) return -1;
  return (int64_t)((((size_t)pt.n * d.h + py - d.pad) * d.w + px - d.pad) * d.c + cc % d.c);
}
float im2col_value(const float* x, uint32_t row, uint32_t cc, const Dims& d) {
  const int64_t at = patch_source(patch_of(row, d), cc, d);
  return at < 0 ? 0.0f : x[at];
}

// src/cpu/ops.zig:12-43 `im2colRows`.
void im2col_rows(const float* src, float* dst, const Dims& d, size_t first, size_t lo, size_t hi) {
  const size_t c = d.c, k = d.k, kc = k * k * c;
  const int64_t w = d.w, pad = d.pad;
  for (size_t index = lo; index < hi; ++index) {
    const Patch pt = patch_of((uint32_t)(first + index), d);
    float* out = dst + index * kc;
    if (d.dilation != 1) {
      for (size_t cc = 0; cc < kc; ++cc) out[cc] = im2col_value(src, (uint32_t)(first + index), (uint32_t)cc, d);
      continue;
    }
    const size_t f = (size_t)std::clamp<int64_t>(pad - (int64_t)pt.left, 0, (int64_t)k);
    const size_t l = (size_t)std::clamp<int64_t>(w + pad - (int64_t)pt.left, 0, (int64_t)k);
    for (size_t ky = 0; ky < k; ++ky) {
      float* line = out + ky * k * c;
      const int64_t y = (int64_t)pt.top + (int64_t)ky - pad;
      if (y < 0 || y >= (int64_t)d.h || l <= f) {
        std::memset(line, 0, k * c * sizeof(float));
        continue;
      }
      std::memset(line, 0, f * c * sizeof(float));
      const size_t from = (((size_t)pt.n * d.h + (size_t)y) * d.w + pt.left + f - d.pad) * c;
      std::memcpy(line + f * c, src + from, (l - f) * c * sizeof(float));
      std::memset(line + l * c, 0, (k - l) * c * sizeof(float));
    }
  }
}
void im2col_range(int threads, const float* x, float* col, const Dims& d, size_t first, size_t count) {
  parallel_for(threads, count, 32, [&](size_t lo, size_t hi) { im2col_rows(x, col, d, first, lo, hi); });
}

constexpr size_t kChunkBytes = 1u << 21;   // src/cpu/ops.zig:54
size_t chunk_rows(const Dims& d) {         // src/cpu/ops.zig:56-59
  return std::min(rows_of(d), std::max<size_t>(1024, kChunkBytes / (patch_len(d) * sizeof(float))));
}

bool conv_is_direct(const Dims& d) {       // src/cpu/ops.zig:84-86
  return d.c == 1 && d.groups == 1 && d.pad == 0 && d.dilation == 1 && d.c_out % lane_count_f32() == 0;
}
size_t direct_origin(const Dims& d, size_t row) {   // src/cpu/ops.zig:89-93
  const size_t ow = out_w(d), oh = out_h(d);
  return ((row / (oh * ow)) * d.h + row / ow % oh * d.stride) * d.w + row % ow * d.stride;
}

// src/cpu/ops.zig:253-285 `col2imPixels`.
void col2im_pixels(const float* src, float* dst, const Dims& d, size_t lo, size_t hi) {
  const size_t c = d.c, kc = patch_len(d);
  const uint32_t oh = out_h(d), ow = out_w(d);
  for (size_t pixel = lo; pixel < hi; ++pixel) {
    const uint32_t y = (uint32_t)(pixel / d.w % d.h + d.pad);
    const uint32_t x = (uint32_t)(pixel % d.w + d.pad);
    const uint32_t n = (uint32_t)(pixel / d.w / d.h);
    float* out = dst + pixel * c;
    for (uint32_t ky = 0; ky < d.k; ++ky) {
      const uint32_t sy = ky * d.dilation;
      if (y < sy || (y - sy) % d.stride != 0) continue;
      const uint32_t oy = (y - sy) / d.stride;
      if (oy >= oh) continue;
      for (uint32_t kx = 0; kx < d.k; ++kx) {
        const uint32_t sx = kx * d.dilation;
        if (x < sx || (x - sx) % d.stride != 0) continue;
        const uint32_t ox = (x - sx) / d.stride;
        if (ox >= ow) continue;
        const float* s = src + (((size_t)n * oh + oy) * ow + ox) * kc + ((size_t)ky * d.k + kx) * c;
        for (size_t i = 0; i < c; ++i) out[i] += s[i];
      }
    }
  }
}

}  // namespace

// =============================================================================================
// Exports
// =============================================================================================
extern "C" {

uint16_t oracle_bf16_encode(float x) {
  uint32_t bits;
  std::memcpy(&bits, &x, 4);
  return (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}
float oracle_bf16_decode(uint16_t h) {
  const uint32_t bits = (uint32_t)h << 16;
  float x;
  std::memcpy(&x, &bits, 4);
  return x;
}
void oracle_bf16_round_array(const float* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = oracle_bf16_decode(oracle_bf16_encode(src[i]));
}
void oracle_bf16_encode_array(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = oracle_bf16_encode(src[i]);
}
void oracle_bf16_decode_array(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = oracle_bf16_decode(src[i]);
}
float oracle_tf32_round(float x) {
  uint32_t bits;
  std::memcpy(&bits, &x, 4);
  if ((bits & 0x7F800000u) != 0x7F800000u) bits += 0x1000u;   // half of the dropped 13 bits, ties away from zero
  bits &= 0xFFFFE000u;
  std::memcpy(&x, &bits, 4);
  return x;
}
void oracle_tf32_round_array(const float* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = oracle_tf32_round(src[i]);
}

void oracle_matmul_naive_f32(size_t m, size_t k, size_t n, const float* a, const float* b, float* out) {
  matmul_naive<float>(m, k, n, a, b, out);
}
void oracle_matmul_naive_f64(size_t m, size_t k, size_t n, const double* a, const double* b, double* out) {
  matmul_naive<double>(m, k, n, a, b, out);
}

void oracle_matmul_tiled_f32(size_t m, size_t k, size_t n, const float* a, const float* b, float* out,
                             int trans_a, int trans_b, int accumulate, int threads) {
  TileConfig cfg;
  cfg.trans_a = trans_a; cfg.trans_b = trans_b; cfg.accumulate = accumulate;
  matmul_tiled<float>(cfg, threads, Problem<float>{m, k, n, a, b, out});
}
void oracle_matmul_tiled_f64(size_t m, size_t k, size_t n, const double* a, const double* b, double* out,
                             int trans_a, int trans_b, int accumulate, int threads) {
  TileConfig cfg;
  cfg.trans_a = trans_a; cfg.trans_b = trans_b; cfg.accumulate = accumulate;
  matmul_tiled<double>(cfg, threads, Problem<double>{m, k, n, a, b, out});
}
void oracle_matmul_tiled_cfg_f32(size_t m, size_t k, size_t n, const float* a, const float* b, float* out,
                                 int trans_a, int trans_b, int accumulate, int threads,
                                 size_t mr, size_t nv, size_t mc, size_t kc, size_t nc) {
  TileConfig cfg;
  cfg.mr = mr; cfg.nv = nv; cfg.mc = mc; cfg.kc = kc; cfg.nc = nc;
  cfg.trans_a = trans_a; cfg.trans_b = trans_b; cfg.accumulate = accumulate;
  matmul_tiled<float>(cfg, threads, Problem<float>{m, k, n, a, b, out});
}
int oracle_split_for(size_t m, size_t k, size_t n, int threads, size_t* parts, size_t* chunk) {
  const Split s = split_for<float>(TileConfig{}, threads, m, k, n);
  if (parts) *parts = s.parts;
  if (chunk) *chunk = s.chunk;
  return s.axis;
}

uint32_t oracle_out_height(const oracle_dims* d) { return out_h(*d); }
uint32_t oracle_out_width(const oracle_dims* d) { return out_w(*d); }

void oracle_im2col_elements(const float* x, float* col, const oracle_dims* d) {
  const size_t kc = patch_len(*d), total = rows_of(*d) * kc;
  for (size_t t = 0; t < total; ++t) col[t] = im2col_value(x, (uint32_t)(t / kc), (uint32_t)(t % kc), *d);
}

// src/gpu/math/conv.zig:93-131 `outputCoord` + `col2imSum` + `col2im`.
void oracle_col2im_elements(const float* dcol, float* dx, const oracle_dims* dp) {
  const Dims& d = *dp;
  const size_t kc = patch_len(d);
  const uint32_t ow = out_w(d), oh = out_h(d);
  const size_t total = (size_t)d.n * d.h * d.w * d.c;
  for (size_t t = 0; t < total; ++t) {
    const uint32_t ch = (uint32_t)(t % d.c), px = (uint32_t)(t / d.c % d.w), py = (uint32_t)(t / d.c / d.w % d.h),
                   pn = (uint32_t)(t / d.c / d.w / d.h);
    float total_v = 0;
    for (uint32_t ky = 0; ky < d.k; ++ky) {
      const uint32_t pos_y = py + d.pad, sh_y = ky * d.dilation;
      if (pos_y < sh_y || (pos_y - sh_y) % d.stride != 0) continue;
      const uint32_t oy = (pos_y - sh_y) / d.stride;
      if (oy >= oh) continue;
      for (uint32_t kx = 0; kx < d.k; ++kx) {
        const uint32_t pos_x = px + d.pad, sh_x = kx * d.dilation;
        if (pos_x < sh_x || (pos_x - sh_x) % d.stride != 0) continue;
        const uint32_t ox = (pos_x - sh_x) / d.stride;
        if (ox >= ow) continue;
        const size_t row = ((size_t)pn * oh + oy) * ow + ox;
        total_v += dcol[row * kc + ((size_t)ky * d.k + kx) * d.c + ch];
      }
    }
    dx[t] += total_v;
  }
}

void oracle_im2col_rows(const float* x, float* col, const oracle_dims* d, size_t first, size_t count, int threads) {
  im2col_range(threads, x, col, *d, first, count);
}
void oracle_col2im_pixels(const float* dcol, float* dx, const oracle_dims* d, int threads) {
  parallel_for(threads, (size_t)d->n * d->h * d->w, 64, [&](size_t lo, size_t hi) { col2im_pixels(dcol, dx, *d, lo, hi); });
}

void oracle_conv_forward(const float* x, const float* w, float* out, const oracle_dims* dp, int threads) {
  const Dims& d = *dp;
  if (conv_is_direct(d)) {
    // src/cpu/ops.zig:99-129: one FMA chain over the k*k taps per output, taps in (ky, kx) order.
    const size_t k = d.k, c_out = d.c_out;
    parallel_for(threads, rows_of(d), 64, [&](size_t lo, size_t hi) {
      for (size_t row = lo; row < hi; ++row) {
        const size_t origin = direct_origin(d, row);
        for (size_t v = 0; v < c_out; ++v) {
          float acc = 0;
          for (size_t ky = 0; ky < k; ++ky)
            for (size_t kx = 0; kx < k; ++kx) acc = std::fma(x[origin + ky * d.w + kx], w[(ky * k + kx) * c_out + v], acc);
          out[row * c_out + v] = acc;
        }
      }
    });
    return;
  }
  const size_t kc = patch_len(d), rows = rows_of(d), chunk = chunk_rows(d);
  std::vector<float> col(chunk * kc);
  TileConfig cfg;
  for (size_t first = 0; first < rows; first += chunk) {
    const size_t count = std::min(chunk, rows - first);
    im2col_range(threads, x, col.data(), d, first, count);
    matmul_tiled<float>(cfg, threads, Problem<float>{count, kc, d.c_out, col.data(), w, out + first * d.c_out});
  }
}

void oracle_conv_input_grad(const float* grad, const float* w, float* dx, const oracle_dims* dp, int threads) {
  const Dims& d = *dp;
  const size_t kc = patch_len(d);
  const size_t per_image = (size_t)out_h(d) * out_w(d);
  const size_t images = std::min<size_t>(d.n, std::max<size_t>(1, kChunkBytes / (per_image * kc * sizeof(float))));
  TileConfig cfg;
  cfg.trans_b = true;
  std::vector<float> dcol(images * per_image * kc);
  for (size_t first = 0; first < d.n; first += images) {
    const size_t count = std::min(images, d.n - first);
    const size_t rows = count * per_image;
    matmul_tiled<float>(cfg, threads, Problem<float>{rows, d.c_out, kc, grad + first * per_image * d.c_out, w, dcol.data()});
    Dims part = d;
    part.n = (uint32_t)count;
    float* dst = dx + first * (size_t)d.h * d.w * d.c;
    parallel_for(threads, count * d.h * d.w, 64, [&](size_t lo, size_t hi) { col2im_pixels(dcol.data(), dst, part, lo, hi); });
  }
}

void oracle_conv_weight_grad(const float* x, const float* grad, float* dw, const oracle_dims* dp, int threads) {
  const Dims& d = *dp;
  if (conv_is_direct(d)) {
    // src/cpu/ops.zig:172-231: each share sums its positions into a private dw in blocks of 64
    // positions (one FMA chain per (tap, channel) per block, added to the private copy per block);
    // the copies are then added to dw in share order.
    const size_t rows = rows_of(d), taps = (size_t)d.k * d.k, c_out = d.c_out, len = taps * c_out;
    const size_t shares = threads <= 1 ? 1 : std::max<size_t>(1, std::min<size_t>((size_t)threads, rows / 256));
    std::vector<float> partial(shares * len, 0.0f);
    const size_t per_share = (rows + shares - 1) / shares;
    parallel_for(threads, shares, 1, [&](size_t lo, size_t hi) {
      for (size_t share = lo; share < hi; ++share) {
        float* mine = partial.data() + share * len;
        const size_t last = std::min(share * per_share + per_share, rows);
        for (size_t first = share * per_share; first < last; first += 64) {
          const size_t count = std::min<size_t>(64, last - first);
          for (size_t v = 0; v < c_out; ++v)
            for (size_t tap = 0; tap < taps; ++tap) {
              const size_t offset = tap / d.k * d.w + tap % d.k;
              float acc = 0;
              for (size_t i = 0; i < count; ++i)
                acc = std::fma(x[direct_origin(d, first + i) + offset], grad[(first + i) * c_out + v], acc);
              mine[tap * c_out + v] += acc;
            }
        }
      }
    });
    for (size_t share = 0; share < shares; ++share)
      for (size_t i = 0; i < len; ++i) dw[i] += partial[share * len + i];
    return;
  }
  const size_t kc = patch_len(d), rows = rows_of(d), chunk = chunk_rows(d);
  TileConfig cfg;
  cfg.trans_a = true;
  cfg.accumulate = true;
  std::vector<float> col(chunk * kc);
  for (size_t first = 0; first < rows; first += chunk) {
    const size_t count = std::min(chunk, rows - first);
    im2col_range(threads, x, col.data(), d, first, count);
    matmul_tiled<float>(cfg, threads, Problem<float>{kc, count, d.c_out, col.data(), grad + first * d.c_out, dw});
  }
}

void oracle_conv_grouped_forward(const float* x, const float* w, float* out, const oracle_dims* dp) {
  const Dims& d = *dp;
  const uint32_t cg = d.c / d.groups, ow = out_w(d), oh = out_h(d);
  const size_t total = rows_of(d) * d.c_out;
  for (size_t t = 0; t < total; ++t) {
    const uint32_t ch = (uint32_t)(t % d.c_out), ox = (uint32_t)(t / d.c_out % ow), oy = (uint32_t)(t / d.c_out / ow % oh),
                   n = (uint32_t)(t / d.c_out / ow / oh);
    const uint32_t base = ch / (d.c_out / d.groups) * cg;
    volatile float total_v = 0;
    for (uint32_t ky = 0; ky < d.k; ++ky) {
      const uint32_t py = oy * d.stride + ky * d.dilation;
      if (py < d.pad || py - d.pad >= d.h) continue;
      for (uint32_t kx = 0; kx < d.k; ++kx) {
        const uint32_t px = ox * d.stride + kx * d.dilation;
        if (px < d.pad || px - d.pad >= d.w) continue;
        const size_t source = (((size_t)n * d.h + py - d.pad) * d.w + px - d.pad) * d.c + base;
        const size_t weights = ((size_t)ky * d.k + kx) * cg;
        for (uint32_t ic = 0; ic < cg; ++ic) {
          const float prod = x[source + ic] * w[(weights + ic) * d.c_out + ch];
          total_v = total_v + prod;
        }
      }
    }
    out[t] = total_v;
  }
}

void oracle_conv_grouped_input_grad(const float* dy, const float* w, float* dx, const oracle_dims* dp) {
  const Dims& d = *dp;
  const uint32_t ow = out_w(d), oh = out_h(d), cg = d.c / d.groups, per_group = d.c_out / d.groups;
  const size_t total = (size_t)d.n * d.h * d.w * d.c;
  for (size_t t = 0; t < total; ++t) {
    const uint32_t ch = (uint32_t)(t % d.c), px = (uint32_t)(t / d.c % d.w), py = (uint32_t)(t / d.c / d.w % d.h),
                   pn = (uint32_t)(t / d.c / d.w / d.h);
    const uint32_t first_out = ch / cg * per_group;
    volatile float total_v = 0;
    for (uint32_t ky = 0; ky < d.k; ++ky) {
      const uint32_t pos_y = py + d.pad, sh_y = ky * d.dilation;
      if (pos_y < sh_y || (pos_y - sh_y) % d.stride != 0) continue;
      const uint32_t oy = (pos_y - sh_y) / d.stride;
      if (oy >= oh) continue;
      for (uint32_t kx = 0; kx < d.k; ++kx) {
        const uint32_t pos_x = px + d.pad, sh_x = kx * d.dilation;
        if (pos_x < sh_x || (pos_x - sh_x) % d.stride != 0) continue;
        const uint32_t ox = (pos_x - sh_x) / d.stride;
        if (ox >= ow) continue;
        const size_t g = (((size_t)pn * oh + oy) * ow + ox) * d.c_out + first_out;
        const size_t wt = (((size_t)ky * d.k + kx) * cg + ch % cg) * d.c_out + first_out;
        for (uint32_t oc = 0; oc < per_group; ++oc) {
          const float prod = dy[g + oc] * w[wt + oc];
          total_v = total_v + prod;
        }
      }
    }
    dx[t] += total_v;
  }
}

void oracle_conv_grouped_weight_grad(const float* x, const float* dy, float* dw, const oracle_dims* dp) {
  const Dims& d = *dp;
  const uint32_t ow = out_w(d), oh = out_h(d), cg = d.c / d.groups;
  const size_t total = (size_t)d.k * d.k * cg * d.c_out;
  for (size_t t = 0; t < total; ++t) {
    const uint32_t oc = (uint32_t)(t % d.c_out), ic = (uint32_t)(t / d.c_out % cg), kx = (uint32_t)(t / d.c_out / cg % d.k),
                   ky = (uint32_t)(t / d.c_out / cg / d.k);
    const uint32_t channel = oc / (d.c_out / d.groups) * cg + ic;
    volatile float total_v = 0;
    for (uint32_t n = 0; n < d.n; ++n)
      for (uint32_t oy = 0; oy < oh; ++oy) {
        const uint32_t py = oy * d.stride + ky * d.dilation;
        if (py < d.pad || py - d.pad >= d.h) continue;
        for (uint32_t ox = 0; ox < ow; ++ox) {
          const uint32_t px = ox * d.stride + kx * d.dilation;
          if (px < d.pad || px - d.pad >= d.w) continue;
          const float prod = x[(((size_t)n * d.h + py - d.pad) * d.w + px - d.pad) * d.c + channel] *
                             dy[(((size_t)n * oh + oy) * ow + ox) * d.c_out + oc];
          total_v = total_v + prod;
        }
      }
    dw[t] += total_v;
  }
}

void oracle_conv_direct_f64(const float* x, const float* w, double* out, const oracle_dims* dp) {
  const Dims& d = *dp;
  const uint32_t oh = out_h(d), ow = out_w(d);
  for (uint32_t n = 0; n < d.n; ++n)
    for (uint32_t oy = 0; oy < oh; ++oy)
      for (uint32_t ox = 0; ox < ow; ++ox)
        for (uint32_t co = 0; co < d.c_out; ++co) {
          double acc = 0;
          for (uint32_t ky = 0; ky < d.k; ++ky)
            for (uint32_t kx = 0; kx < d.k; ++kx) {
              const int64_t iy = (int64_t)oy * d.stride + (int64_t)ky * d.dilation - d.pad;
              const int64_t ix = (int64_t)ox * d.stride + (int64_t)kx * d.dilation - d.pad;
              if (iy < 0 || ix < 0 || iy >= (int64_t)d.h || ix >= (int64_t)d.w) continue;
              for (uint32_t ci = 0; ci < d.c; ++ci)
                acc += (double)x[(((size_t)n * d.h + iy) * d.w + ix) * d.c + ci] *
                       (double)w[(((size_t)ky * d.k + kx) * d.c + ci) * d.c_out + co];
            }
          out[(((size_t)n * oh + oy) * ow + ox) * d.c_out + co] = acc;
        }
}

void oracle_reorder_oihw(const float* w, float* wt, size_t m, size_t c, size_t kh, size_t kw) {
  const size_t khkw = kh * kw;
  for (size_t item = 0; item < c * khkw; ++item) {
    const size_t tap = item / c, ic = item % c;
    for (size_t oc = 0; oc < m; ++oc) wt[item * m + oc] = w[(oc * c + ic) * khkw + tap];
  }
}

void oracle_convolve_nhwc(const float* x, const float* w_oihw, const float* bias, float* out,
                          const oracle_dims* d, int threads) {
  std::vector<float> wt((size_t)d->k * d->k * d->c * d->c_out);
  oracle_reorder_oihw(w_oihw, wt.data(), d->c_out, d->c, d->k, d->k);
  oracle_conv_forward(x, wt.data(), out, d, threads);
  if (bias) {
    const size_t len = rows_of(*d) * d->c_out;
    for (size_t i = 0; i < len; ++i) out[i] += bias[i % d->c_out];
  }
}

void oracle_convolve_nchw(const float* x, const float* w, const float* bias, float* out,
                          size_t n, size_t c, size_t h, size_t width, size_t m, size_t kh, size_t kw,
                          size_t groups, size_t stride, size_t pad, size_t dilation, int threads) {
  const size_t oh = (h + 2 * pad - dilation * (kh - 1) - 1) / stride + 1;
  const size_t ow = (width + 2 * pad - dilation * (kw - 1) - 1) / stride + 1;
  if (groups == 1) {
    // src/onnx/runtime.zig:786-801 + planarColumns :666-700: col is (c*kh*kw) x (oh*ow), out = w * col per image.
    const size_t taps = c * kh * kw, positions = oh * ow;
    std::vector<float> col(taps * positions);
    TileConfig cfg;
    for (size_t b = 0; b < n; ++b) {
      const float* xi = x + b * c * h * width;
      for (size_t ic = 0; ic < c; ++ic)
        for (size_t ky = 0; ky < kh; ++ky)
          for (size_t kx = 0; kx < kw; ++kx) {
            float* line = col.data() + ((ic * kh + ky) * kw + kx) * positions;
            for (size_t oy = 0; oy < oh; ++oy) {
              const size_t iy = oy * stride + ky * dilation;
              for (size_t ox = 0; ox < ow; ++ox) {
                const size_t ix = ox * stride + kx * dilation;
                const bool inside = iy >= pad && iy - pad < h && ix >= pad && ix - pad < width;
                line[oy * ow + ox] = inside ? xi[(ic * h + iy - pad) * width + ix - pad] : 0.0f;
              }
            }
          }
      float* image = out + b * m * positions;
      matmul_tiled<float>(cfg, threads, Problem<float>{m, taps, positions, w, col.data(), image});
      if (bias)
        for (size_t ch = 0; ch < m; ++ch)
          for (size_t i = 0; i < positions; ++i) image[ch * positions + i] += bias[ch];
    }
    return;
  }
  const size_t pg = c / groups, m_per_group = m / groups;
  for (size_t row = 0; row < n * m * oh; ++row) {
    const size_t b = row / (m * oh), oc = row / oh % m, oy = row % oh, g = oc / m_per_group;
    for (size_t ox = 0; ox < ow; ++ox) {
      volatile float total = bias ? bias[oc] : 0.0f;
      for (size_t ic = 0; ic < pg; ++ic) {
        const size_t channel = g * pg + ic;
        for (size_t ky = 0; ky < kh; ++ky) {
          const size_t iy = oy * stride + ky * dilation;
          if (iy < pad || iy - pad >= h) continue;
          for (size_t kx = 0; kx < kw; ++kx) {
            const size_t ix = ox * stride + kx * dilation;
            if (ix < pad || ix - pad >= width) continue;
            const float prod = x[((b * c + channel) * h + iy - pad) * width + ix - pad] * w[((oc * pg + ic) * kh + ky) * kw + kx];
            total = total + prod;
          }
        }
      }
      out[((b * m + oc) * oh + oy) * ow + ox] = total;
    }
  }
}

void oracle_onnx_matmul(const float* x, const float* y, float* out, size_t batch, size_t weight_batch,
                        size_t m, size_t k, size_t n, int threads) {
  TileConfig cfg;
  for (size_t b = 0; b < batch; ++b) {
    const float* w = y + (weight_batch == 1 ? 0 : b) * k * n;
    if (m != 0 && k != 0 && n != 0) {
      matmul_tiled<float>(cfg, threads, Problem<float>{m, k, n, x + b * m * k, w, out + b * m * n});
    } else {
      std::fill(out + b * m * n, out + (b + 1) * m * n, 0.0f);
    }
  }
}

void oracle_onnx_gemm(const float* x, const float* y, const float* c, float* out, size_t m, size_t k, size_t n,
                      int trans_a, int trans_b, float alpha, float beta, int threads) {
  std::vector<float> lhs, rhs;
  if (trans_a) {   // x stored (k, m)
    lhs.resize(m * k);
    for (size_t i = 0; i < k; ++i)
      for (size_t j = 0; j < m; ++j) lhs[j * k + i] = x[i * m + j];
    x = lhs.data();
  }
  if (trans_b) {   // y stored (n, k)
    rhs.resize(k * n);
    for (size_t i = 0; i < n; ++i)
      for (size_t j = 0; j < k; ++j) rhs[j * n + i] = y[i * k + j];
    y = rhs.data();
  }
  oracle_onnx_matmul(x, y, out, 1, 1, m, k, n, threads);
  for (size_t i = 0; i < m * n; ++i) out[i] *= alpha;
  if (c)
    for (size_t i = 0; i < m; ++i)
      for (size_t j = 0; j < n; ++j) out[i * n + j] += c[j] * beta;
}

void oracle_relu(float* v, size_t n) {
  for (size_t i = 0; i < n; ++i) v[i] = v[i] > 0 ? v[i] : 0.0f;
}

void oracle_bias_act(float* out, const float* bias, size_t rows, size_t cols, int relu) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      float v = out[r * cols + c];
      if (bias) v += bias[c];
      if (relu) v = v > 0 ? v : 0.0f;
      out[r * cols + c] = v;
    }
}

void oracle_average_grads(float* grads, size_t replicas, size_t len) {
  const float scale = 1.0f / (float)replicas;
  for (size_t i = 0; i < len; ++i) {
    float total = grads[i];   // replica 0's buffer is the running sum (src/nn/replicas.zig:76-79)
    for (size_t r = 1; r < replicas; ++r) total += grads[r * len + i];
    total *= scale;
    for (size_t r = 0; r < replicas; ++r) grads[r * len + i] = total;
  }
}

int oracle_host_threads(void) {
  const unsigned n = std::thread::hardware_concurrency();
  return n == 0 ? 1 : (int)n;
}
int oracle_vector_lanes(void) { return (int)lane_count_f32(); }

}  // extern "C"
