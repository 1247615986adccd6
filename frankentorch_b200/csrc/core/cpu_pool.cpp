// CPU thread-width policy and the parallel forms of the CPU reference kernels.
//
// Behaviour of ft-kernel-cpu/src/pool.rs (:69 physical_cores, :119 auto_width =
// min(16, physical cores), :139 resolve_width, :166 configure_global_pool): the width is
// opt-in - unset means serial - and "auto" caps at 16 because the reference measured its
// lanes getting slower beyond that.  It is decided once; a second configuration attempt
// reports what is in force instead of changing it.
//
// The parallel kernels split work so that no reduction is ever divided between threads
// (rows of a matrix, fixed sub-trees of the pairwise sum): the result has the same bits
// as the serial kernel, whatever the width and whatever the size gate
// (ft-kernel-cpu/src/lib.rs:21-40, :4120; tests/threshold_serial_parallel_equivalence.rs).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <set>
#include <sstream>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#define FTC_API extern "C" __attribute__((visibility("default")))

namespace {

std::mutex g_mu;
int g_width = 1;             // 1 = serial
bool g_configured = false;
int64_t g_par_min_work = 1 << 15;   // below this many elements of work a kernel stays serial
int g_target_workers = 0;           // 0 = split into one chunk per pool thread; n = into about n chunks

// Distinct (physical id, core id) pairs of /proc/cpuinfo; falls back to the logical count.
int physical_cores() {
  std::ifstream f("/proc/cpuinfo");
  std::set<std::pair<int, int>> cores;
  std::string line;
  int phys = -1, core = -1;
  while (std::getline(f, line)) {
    if (line.rfind("physical id", 0) == 0) phys = std::atoi(line.substr(line.find(':') + 1).c_str());
    if (line.rfind("core id", 0) == 0) core = std::atoi(line.substr(line.find(':') + 1).c_str());
    if (line.empty()) {
      if (phys >= 0 && core >= 0) cores.insert({phys, core});
      phys = core = -1;
    }
  }
  if (phys >= 0 && core >= 0) cores.insert({phys, core});
  if (!cores.empty()) return (int)cores.size();
  const unsigned n = std::thread::hardware_concurrency();
  return n ? (int)n : 1;
}

template <typename F>
void parallel_rows(int64_t rows, int64_t work_per_row, F fn) {
  int w = g_width;
  if (w > 1 && g_target_workers > 0) w = g_target_workers;
  if (w <= 1 || rows < 2 || rows * work_per_row < g_par_min_work) {
    fn(0, rows);
    return;
  }
  if (w > rows) w = (int)rows;
  std::vector<std::thread> th;
  const int64_t per = (rows + w - 1) / w;
  for (int t = 0; t < w; ++t) {
    const int64_t a = t * per, b = std::min(rows, a + per);
    if (a >= b) break;
    th.emplace_back([=] { fn(a, b); });
  }
  for (auto& t : th) t.join();
}

double pairwise(const double* x, int64_t n) {
  if (n <= 128) {
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += x[i];
    return s;
  }
  const int64_t mid = n / 2;
  return pairwise(x, mid) + pairwise(x + mid, n - mid);
}
// The same tree, with the two halves of the top `depth` levels summed by different threads.
double pairwise_par(const double* x, int64_t n, int depth) {
  if (depth <= 0 || n <= 128) return pairwise(x, n);
  const int64_t mid = n / 2;
  double left = 0.0;
  std::thread t([&] { left = pairwise_par(x, mid, depth - 1); });
  const double right = pairwise_par(x + mid, n - mid, depth - 1);
  t.join();
  return left + right;
}

}  // namespace

// spec: "" / null = leave serial, "auto" = min(16, physical cores), "<n>" = n (>= 1).
// Returns the width in force; *changed = 1 when this call set it.  Malformed specs return -1.
FTC_API int ftc_pool_configure(const char* spec, int* changed) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (changed) *changed = 0;
  if (g_configured) return g_width;
  if (!spec || !*spec) return g_width;
  int w;
  if (std::strcmp(spec, "auto") == 0) {
    w = std::min(16, physical_cores());
  } else {
    char* end = nullptr;
    const long v = std::strtol(spec, &end, 10);
    if (!end || *end || v < 1 || v > 4096) return -1;
    w = (int)v;
  }
  g_width = std::max(1, w);
  g_configured = true;
  if (changed) *changed = 1;
  return g_width;
}
FTC_API int ftc_pool_width() { return g_width; }
FTC_API int ftc_pool_physical_cores() { return physical_cores(); }
FTC_API int ftc_pool_auto_width() { return std::min(16, physical_cores()); }
// Test hook: forget the configuration (the process-wide policy is otherwise decided once).
FTC_API void ftc_pool_reset_for_tests() {
  std::lock_guard<std::mutex> lock(g_mu);
  g_width = 1;
  g_configured = false;
}
// Size gate below which kernels stay serial (set_parallel_target_workers / PAR_MIN_FLOPS analogue).
FTC_API int64_t ftc_pool_set_min_work(int64_t elems) {
  const int64_t old = g_par_min_work;
  if (elems >= 0) g_par_min_work = elems;
  return old;
}

// Number of chunks a row-parallel kernel is cut into (0 = the pool width).  Returns the previous value, so a
// measurement can flip it inside one process and restore it.  Every row is computed by one thread whatever the
// split, so results do not depend on it.
FTC_API int ftc_pool_set_target_workers(int workers) {
  const int old = g_target_workers;
  if (workers >= 0 && workers <= 4096) g_target_workers = workers;
  return old;
}
FTC_API int ftc_pool_target_workers() { return g_target_workers; }

FTC_API double ftc_pairwise_sum_par(const double* x, int64_t n) {
  int w = g_width, depth = 0;
  while ((1 << depth) < w) ++depth;
  if (w <= 1 || n < g_par_min_work) depth = 0;
  return pairwise_par(x, n, depth);
}

// y[m,n] = x[m,k] . w[n,k]^T + b[n], rows of y split between threads (K is never split)
FTC_API void ftc_linear_f64_par(const double* x, const double* w, const double* b, double* y, int64_t m,
                                int64_t k, int64_t n) {
  parallel_rows(m, k * n, [=](int64_t r0, int64_t r1) {
    for (int64_t i = r0; i < r1; ++i)
      for (int64_t j = 0; j < n; ++j) {
        double s = 0.0;
        const double* xr = x + i * k;
        const double* wr = w + j * k;
        for (int64_t p = 0; p < k; ++p) s += xr[p] * wr[p];
        y[i * n + j] = s + (b ? b[j] : 0.0);
      }
  });
}

// Two-pass LayerNorm, rows split between threads
FTC_API void ftc_layer_norm_f64_par(const double* x, const double* g, const double* b, double* y,
                                    int64_t rows, int64_t cols, double eps) {
  parallel_rows(rows, cols, [=](int64_t r0, int64_t r1) {
    for (int64_t r = r0; r < r1; ++r) {
      const double* xr = x + r * cols;
      double mean = 0.0;
      for (int64_t c = 0; c < cols; ++c) mean += xr[c];
      mean /= (double)cols;
      double var = 0.0;
      for (int64_t c = 0; c < cols; ++c) var += (xr[c] - mean) * (xr[c] - mean);
      const double rstd = 1.0 / std::sqrt(var / (double)cols + eps);
      for (int64_t c = 0; c < cols; ++c)
        y[r * cols + c] = (xr[c] - mean) * rstd * (g ? g[c] : 1.0) + (b ? b[c] : 0.0);
    }
  });
}

// AdamW single pass (ft-optim/src/lib.rs:1040-1054), elements split between threads
FTC_API void ftc_adamw_f64_par(double* p, const double* g, double* m, double* v, int64_t n, double lr,
                               double b1, double b2, double eps, double wd, int64_t step) {
  const double bc1 = 1.0 - std::pow(b1, (double)step), bc2 = 1.0 - std::pow(b2, (double)step);
  parallel_rows(n, 1, [=](int64_t a, int64_t e) {
    for (int64_t i = a; i < e; ++i) {
      m[i] = b1 * m[i] + (1.0 - b1) * g[i];
      v[i] = b2 * v[i] + (1.0 - b2) * g[i] * g[i];
      const double mh = m[i] / bc1, vh = v[i] / bc2;
      p[i] -= p[i] * lr * wd + lr * mh / (std::sqrt(vh) + eps);
    }
  });
}

// ---- blocked scaled dot-product attention with a tunable query-row tile ------------------------------
// Counterpart of the reference's `sdpa_forward_f32` tile controls (ft-kernel-cpu/src/lib.rs:4912-4990):
// the work items are (batch*head, block of BR query rows); BR is a process-wide setting with a fixed
// default of 64, a programmatic setter (so one process can sweep it) and an environment override read once
// (FT_SDPA_BR, 8..512); 0 selects the adaptive rule: 128 when the heads alone fill the pool or when
// heads x blocks stays above four tasks per thread, else 64.  Every output row is computed by one thread
// with the same loop as the serial oracle, so the result is bit-identical for every BR and every pool width:
// BR can only change scheduling.
namespace {
std::atomic<int> g_sdpa_br{64};
std::once_flag g_sdpa_env_once;
constexpr int SDPA_BR_SMALL = 64, SDPA_BR_LARGE = 128, SDPA_TASKS_PER_THREAD = 4;

void sdpa_env_init() {
  std::call_once(g_sdpa_env_once, [] {
    if (const char* e = std::getenv("FT_SDPA_BR")) {
      char* end = nullptr;
      const long b = std::strtol(e, &end, 10);
      if (end != e && *end == 0 && b >= 8 && b <= 512) g_sdpa_br.store((int)b);
    }
  });
}
int sdpa_br_pick(int64_t sq, int64_t num_bh, int threads) {
  threads = std::max(1, threads);
  if (num_bh >= threads) return SDPA_BR_LARGE;
  const int64_t blocks = (sq + SDPA_BR_LARGE - 1) / SDPA_BR_LARGE;
  return num_bh * blocks >= (int64_t)SDPA_TASKS_PER_THREAD * threads ? SDPA_BR_LARGE : SDPA_BR_SMALL;
}
void sdpa_rows(const double* q, const double* k, const double* v, double* o, int64_t r0, int64_t r1, int64_t sk,
               int64_t d, double scale, int causal, std::vector<double>& p) {
  for (int64_t i = r0; i < r1; ++i) {
    double m = -INFINITY;
    const int64_t lim = causal ? std::min<int64_t>(sk, i + 1) : sk;
    for (int64_t j = 0; j < lim; ++j) {
      double s = 0.0;
      for (int64_t e = 0; e < d; ++e) s += q[i * d + e] * k[j * d + e];
      p[j] = s * scale;
      m = std::max(m, p[j]);
    }
    double z = 0.0;
    for (int64_t j = 0; j < lim; ++j) {
      p[j] = std::exp(p[j] - m);
      z += p[j];
    }
    for (int64_t e = 0; e < d; ++e) {
      double s = 0.0;
      for (int64_t j = 0; j < lim; ++j) s += p[j] * v[j * d + e];
      o[i * d + e] = s / z;
    }
  }
}
}  // namespace

// br: 0 = adaptive, otherwise clamped to [8, 512].  Returns the value now stored.
FTC_API int ftc_set_sdpa_br(int br) {
  sdpa_env_init();
  if (br != 0) br = std::min(512, std::max(8, br));
  g_sdpa_br.store(br);
  return br;
}
FTC_API int ftc_get_sdpa_br() {
  sdpa_env_init();
  return g_sdpa_br.load();
}
// The tile the kernel would use for this problem (the stored value, or the adaptive choice when it is 0).
FTC_API int ftc_sdpa_br_for(int64_t sq, int64_t num_bh) {
  sdpa_env_init();
  const int b = g_sdpa_br.load();
  return b != 0 ? b : sdpa_br_pick(sq, num_bh, g_width);
}
// q, k, v, o: [num_bh, s, d] contiguous.  Work items (bh, row block) are dealt to the pool in order.
FTC_API void ftc_sdpa_f64_blocked(const double* q, const double* k, const double* v, double* o, int64_t num_bh,
                                  int64_t sq, int64_t sk, int64_t d, double scale, int causal) {
  const int br = ftc_sdpa_br_for(sq, num_bh);
  const int64_t blocks = (sq + br - 1) / br, items = num_bh * blocks;
  parallel_rows(items, (int64_t)br * sk * d * 2, [=](int64_t i0, int64_t i1) {
    std::vector<double> p((size_t)sk);
    for (int64_t it = i0; it < i1; ++it) {
      const int64_t bh = it / blocks, blk = it % blocks;
      const int64_t r0 = blk * br, r1 = std::min(sq, r0 + br);
      sdpa_rows(q + bh * sq * d, k + bh * sk * d, v + bh * sk * d, o + bh * sq * d, r0, r1, sk, d, scale, causal, p);
    }
  });
}
