// Host runtime of frankentorch_b200 (C ABI, loaded through ctypes).
//
//  * TapeCore      - graph store + deterministic backward scheduler of the
//                    Deterministic Autograd Contract: reachability DFS, dependency
//                    counts, max-heap ready queue keyed by node id (highest id
//                    first), telemetry.  Behaviour follows ft-autograd/src/lib.rs
//                    (:826-873 ready queue, :11724-11830 backward loop, :19498
//                    compute_reachable, :19669 compute_dependencies, :19839
//                    complete_dependency).
//  * EvidenceLedger- bounded provenance ledger (ft-runtime/src/lib.rs:46-55): soft cap
//                    32,768 entries; when exceeded keep entry 0 plus the newest half.
//  * FNV-1a 64     - deterministic fingerprints (ft-core/src/lib.rs:660-679,
//                    ft-dispatch/src/lib.rs:1144 digest64).
//  * PRNGs         - xoshiro256++ (session RNG) and the 64-bit LCG of the data loader
//                    (ft-data/src/lib.rs:255-272: state*6364136223846793005+1, >>33).
//  * Dispatch      - key-set validation and strict/hardened resolution
//                    (ft-dispatch/src/lib.rs:520-647, :1361-1393).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <queue>
#include <string>
#include <vector>

#define FTC_API extern "C" __attribute__((visibility("default")))

// ================================================================================ TapeCore
namespace {

struct TapeNode {
  std::vector<int64_t> inputs;
  uint8_t requires_grad;
  uint8_t is_leaf;
};

struct TapeCore {
  std::vector<TapeNode> nodes;
  bool consumed = false;
  int64_t consumed_boundary = 0;
};

enum : int64_t {
  FTC_ERR_UNKNOWN_NODE = -1,
  FTC_ERR_ROOT_NO_GRAD = -2,
  FTC_ERR_GRAPH_CONSUMED = -3,
  FTC_ERR_DEP_UNDERFLOW = -4,
  FTC_ERR_BAD_INPUT = -5,
};

}  // namespace

FTC_API void* ftc_tape_new() { return new TapeCore(); }
FTC_API void ftc_tape_free(void* t) { delete static_cast<TapeCore*>(t); }
FTC_API int64_t ftc_tape_len(void* t) { return (int64_t) static_cast<TapeCore*>(t)->nodes.size(); }

// Append a node; ids are append-order indices.  Inputs must already exist.
FTC_API int64_t ftc_tape_add_node(void* tp, const int64_t* inputs, int n_inputs, int requires_grad,
                                  int is_leaf) {
  TapeCore* t = static_cast<TapeCore*>(tp);
  const int64_t id = (int64_t)t->nodes.size();
  TapeNode n;
  n.inputs.reserve(n_inputs);
  for (int i = 0; i < n_inputs; ++i) {
    if (inputs[i] < 0 || inputs[i] >= id) return FTC_ERR_BAD_INPUT;
    n.inputs.push_back(inputs[i]);
  }
  n.requires_grad = requires_grad ? 1 : 0;
  n.is_leaf = is_leaf ? 1 : 0;
  t->nodes.push_back(std::move(n));
  return id;
}

FTC_API int ftc_tape_set_requires_grad(void* tp, int64_t id, int flag) {
  TapeCore* t = static_cast<TapeCore*>(tp);
  if (id < 0 || id >= (int64_t)t->nodes.size()) return -1;
  t->nodes[id].requires_grad = flag ? 1 : 0;
  return 0;
}

// Drop every node with id >= boundary (ids below stay valid).
FTC_API int64_t ftc_tape_truncate(void* tp, int64_t boundary) {
  TapeCore* t = static_cast<TapeCore*>(tp);
  if (boundary < 0) boundary = 0;
  if (boundary < (int64_t)t->nodes.size()) t->nodes.resize(boundary);
  if (t->consumed_boundary > boundary) t->consumed_boundary = boundary;
  if (t->consumed_boundary == 0) t->consumed = false;
  return (int64_t)t->nodes.size();
}

FTC_API void ftc_tape_mark_consumed(void* tp) {
  TapeCore* t = static_cast<TapeCore*>(tp);
  t->consumed = true;
  t->consumed_boundary = (int64_t)t->nodes.size();
}
FTC_API int ftc_tape_is_consumed(void* tp, int64_t root) {
  TapeCore* t = static_cast<TapeCore*>(tp);
  return (t->consumed && root < t->consumed_boundary) ? 1 : 0;
}

// Plan a backward pass from `root`.
//   order_out : capacity = number of nodes; receives the execution order
//   deps_out  : capacity = number of nodes; dependency snapshot (reachable consumers per node)
//   stats_out : [queue_pushes, queue_pops, max_queue_len]
// Returns the number of executed nodes, or a negative error code.
FTC_API int64_t ftc_tape_schedule(void* tp, int64_t root, int check_consumed, int64_t* order_out,
                                  int64_t* deps_out, int64_t* stats_out) {
  TapeCore* t = static_cast<TapeCore*>(tp);
  const int64_t n = (int64_t)t->nodes.size();
  if (check_consumed && t->consumed && root < t->consumed_boundary) return FTC_ERR_GRAPH_CONSUMED;
  if (root < 0 || root >= n) return FTC_ERR_UNKNOWN_NODE;
  if (!t->nodes[root].requires_grad) return FTC_ERR_ROOT_NO_GRAD;

  std::vector<uint8_t> reachable(n, 0);
  std::vector<int64_t> stack{root};
  while (!stack.empty()) {
    const int64_t v = stack.back();
    stack.pop_back();
    if (reachable[v]) continue;
    reachable[v] = 1;
    for (int64_t in : t->nodes[v].inputs) stack.push_back(in);
  }
  std::vector<int64_t> pending(n, 0);
  for (int64_t i = 0; i < n; ++i) {
    if (!reachable[i]) continue;
    for (int64_t in : t->nodes[i].inputs) pending[in] += 1;
  }
  for (int64_t i = 0; i < n; ++i) deps_out[i] = pending[i];

  std::priority_queue<int64_t> queue;  // max-heap: highest node id first
  int64_t pushes = 0, pops = 0, max_len = 0, count = 0;
  queue.push(root);
  pushes = 1;
  max_len = 1;
  while (!queue.empty()) {
    const int64_t v = queue.top();
    queue.pop();
    ++pops;
    order_out[count++] = v;
    for (int64_t in : t->nodes[v].inputs) {
      if (pending[in] == 0) return FTC_ERR_DEP_UNDERFLOW;
      if (--pending[in] == 0) {
        queue.push(in);
        ++pushes;
        max_len = std::max<int64_t>(max_len, (int64_t)queue.size());
      }
    }
  }
  stats_out[0] = pushes;
  stats_out[1] = pops;
  stats_out[2] = max_len;
  return count;
}

// ================================================================================ Ledger
namespace {
struct LedgerEntry {
  int64_t ts_unix_ms;
  int kind;
  std::string summary;
};
struct Ledger {
  std::vector<LedgerEntry> entries;
  size_t soft_cap = 32768;
  std::mutex mu;
  int64_t total_recorded = 0;
};
int64_t now_ms() {
  using namespace std::chrono;
  return duration_cast<milliseconds>(system_clock::now().time_since_epoch()).count();
}
}  // namespace

FTC_API void* ftc_ledger_new(int64_t soft_cap) {
  Ledger* l = new Ledger();
  if (soft_cap > 1) l->soft_cap = (size_t)soft_cap;
  return l;
}
FTC_API void ftc_ledger_free(void* l) { delete static_cast<Ledger*>(l); }
FTC_API int64_t ftc_ledger_record(void* lp, int kind, const char* summary, int64_t ts_ms) {
  Ledger* l = static_cast<Ledger*>(lp);
  std::lock_guard<std::mutex> g(l->mu);
  l->entries.push_back(LedgerEntry{ts_ms >= 0 ? ts_ms : now_ms(), kind, summary ? summary : ""});
  l->total_recorded += 1;
  if (l->entries.size() > l->soft_cap) {
    // keep the anchor (entry 0) and the newest half of the cap
    const size_t keep = l->soft_cap / 2;
    std::vector<LedgerEntry> kept;
    kept.reserve(keep + 1);
    kept.push_back(std::move(l->entries.front()));
    const size_t start = l->entries.size() - keep;
    for (size_t i = std::max<size_t>(start, 1); i < l->entries.size(); ++i)
      kept.push_back(std::move(l->entries[i]));
    l->entries.swap(kept);
  }
  return (int64_t)l->entries.size();
}
FTC_API int64_t ftc_ledger_len(void* lp) {
  Ledger* l = static_cast<Ledger*>(lp);
  std::lock_guard<std::mutex> g(l->mu);
  return (int64_t)l->entries.size();
}
FTC_API int64_t ftc_ledger_total(void* lp) { return static_cast<Ledger*>(lp)->total_recorded; }
// Copies entry `i` into the caller's buffer; returns the summary length (may exceed cap).
FTC_API int64_t ftc_ledger_get(void* lp, int64_t i, int64_t* ts_out, int* kind_out, char* buf,
                               int64_t cap) {
  Ledger* l = static_cast<Ledger*>(lp);
  std::lock_guard<std::mutex> g(l->mu);
  if (i < 0 || i >= (int64_t)l->entries.size()) return -1;
  const LedgerEntry& e = l->entries[i];
  *ts_out = e.ts_unix_ms;
  *kind_out = e.kind;
  const int64_t len = (int64_t)e.summary.size();
  if (buf && cap > 0) {
    const int64_t c = std::min<int64_t>(len, cap - 1);
    std::memcpy(buf, e.summary.data(), (size_t)c);
    buf[c] = 0;
  }
  return len;
}
FTC_API void ftc_ledger_clear(void* lp) {
  Ledger* l = static_cast<Ledger*>(lp);
  std::lock_guard<std::mutex> g(l->mu);
  l->entries.clear();
}

// ================================================================================ FNV-1a
FTC_API uint64_t ftc_fnv1a64(const uint8_t* data, int64_t len, uint64_t seed) {
  uint64_t h = seed ? seed : 0xcbf29ce484222325ull;
  for (int64_t i = 0; i < len; ++i) {
    h ^= (uint64_t)data[i];
    h *= 0x00000100000001b3ull;
  }
  return h;
}

// ================================================================================ PRNGs
namespace {
inline uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
inline uint64_t splitmix64(uint64_t& s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
inline uint64_t xoshiro_next(uint64_t* s) {
  const uint64_t result = rotl(s[0] + s[3], 23) + s[0];
  const uint64_t t = s[1] << 17;
  s[2] ^= s[0];
  s[3] ^= s[1];
  s[1] ^= s[2];
  s[0] ^= s[3];
  s[2] ^= t;
  s[3] = rotl(s[3], 45);
  return result;
}
}  // namespace

// state: 4 x u64.  Seeding expands a 64-bit seed with splitmix64.
FTC_API void ftc_xoshiro_seed(uint64_t* state, uint64_t seed) {
  uint64_t s = seed;
  for (int i = 0; i < 4; ++i) state[i] = splitmix64(s);
}
FTC_API uint64_t ftc_xoshiro_next_u64(uint64_t* state) { return xoshiro_next(state); }
// uniform doubles in [0,1): top 53 bits
FTC_API void ftc_xoshiro_fill_uniform(uint64_t* state, double* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = (double)(xoshiro_next(state) >> 11) * (1.0 / 9007199254740992.0);
}
// standard normals by Box-Muller (two uniforms per pair; cosine branch then sine branch)
FTC_API void ftc_xoshiro_fill_normal(uint64_t* state, double* out, int64_t n) {
  const double two_pi = 6.283185307179586476925286766559;
  int64_t i = 0;
  while (i < n) {
    double u1 = (double)(xoshiro_next(state) >> 11) * (1.0 / 9007199254740992.0);
    double u2 = (double)(xoshiro_next(state) >> 11) * (1.0 / 9007199254740992.0);
    if (u1 < 1e-300) u1 = 1e-300;
    const double r = std::sqrt(-2.0 * std::log(u1));
    out[i++] = r * std::cos(two_pi * u2);
    if (i < n) out[i++] = r * std::sin(two_pi * u2);
  }
}
// 64-bit LCG of the data loader: state = state*6364136223846793005 + 1; value = state >> 33
FTC_API uint64_t ftc_lcg_next(uint64_t* state) {
  *state = (*state) * 6364136223846793005ull + 1ull;
  return (*state) >> 33;
}
// Fisher-Yates from the top index down, draw = next() % (i+1)
FTC_API void ftc_lcg_shuffle(uint64_t* state, int64_t* idx, int64_t n) {
  for (int64_t i = n - 1; i > 0; --i) {
    const uint64_t j = ftc_lcg_next(state) % (uint64_t)(i + 1);
    std::swap(idx[i], idx[(int64_t)j]);
  }
}

// ================================================================================ Dispatch
namespace {
enum Key : int {
  K_UNDEFINED = 0,
  K_BACKEND_SELECT = 1,
  K_COMPOSITE_IMPLICIT = 2,
  K_COMPOSITE_EXPLICIT = 3,
  K_CPU = 4,
  K_AUTOGRAD_CPU = 5,
  K_SM100 = 6,
  K_AUTOGRAD_SM100 = 7,
};
inline uint64_t bit(int k) { return 1ull << k; }
const uint64_t KNOWN_MASK = bit(1) | bit(2) | bit(3) | bit(4) | bit(5) | bit(6) | bit(7);
}  // namespace

// Resolution outcome codes
//   0 ok; 1 empty set; 2 no type key; 3 no backend key; 4 unknown bits;
//   5 autograd key without its backend; 6 strict mode forbids composite/backend fallback;
//   7 resolved key / backend key drifted to an incompatible pair
// out[0]=selected key, out[1]=backend key, out[2]=effective key, out[3]=fallback_used
FTC_API int ftc_dispatch_resolve(uint64_t bits, int hardened, int* out) {
  if (bits & ~KNOWN_MASK) return 4;
  if (bits == 0) return 1;
  if ((bits & bit(K_AUTOGRAD_CPU)) && !(bits & bit(K_CPU))) return 5;
  if ((bits & bit(K_AUTOGRAD_SM100)) && !(bits & bit(K_SM100))) return 5;
  // type priority: autograd keys, composites, backends, backend-select
  static const int type_prio[] = {K_AUTOGRAD_SM100, K_AUTOGRAD_CPU, K_COMPOSITE_EXPLICIT,
                                  K_COMPOSITE_IMPLICIT, K_SM100, K_CPU, K_BACKEND_SELECT};
  static const int backend_prio[] = {K_SM100, K_CPU};
  int selected = K_UNDEFINED, backend = K_UNDEFINED;
  for (int k : type_prio)
    if (bits & bit(k)) {
      selected = k;
      break;
    }
  if (selected == K_UNDEFINED) return 2;
  for (int k : backend_prio)
    if (bits & bit(k)) {
      backend = k;
      break;
    }
  if (backend == K_UNDEFINED) return 3;
  int effective = selected, fallback = 0;
  switch (selected) {
    case K_AUTOGRAD_CPU:
    case K_CPU:
    case K_AUTOGRAD_SM100:
    case K_SM100:
      break;
    default:
      if (!hardened) return 6;
      effective = backend;
      fallback = 1;
  }
  const bool autograd_ok = (effective == K_AUTOGRAD_CPU && backend == K_CPU) ||
                           (effective == K_AUTOGRAD_SM100 && backend == K_SM100);
  if (effective != backend && !autograd_ok) return 7;
  out[0] = selected;
  out[1] = backend;
  out[2] = effective;
  out[3] = fallback;
  return 0;
}

// ================================================================================ CPU reference kernels
// Plain restatements of the reference's CPU math, used as the oracle for the CUDA
// kernels and as the timed CPU baseline.  Summation order is fixed (serial over the
// reduction index; pairwise tree for `ftc_pairwise_sum`).

// Pairwise summation: midpoint split down to 128-element leaves
// (ft-kernel-cpu/src/lib.rs:4105).
static double pairwise(const double* x, int64_t n) {
  if (n <= 128) {
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += x[i];
    return s;
  }
  const int64_t mid = n / 2;
  return pairwise(x, mid) + pairwise(x + mid, n - mid);
}
FTC_API double ftc_pairwise_sum(const double* x, int64_t n) { return pairwise(x, n); }

// y[m,n] = x[m,k] . w[n,k]^T + b[n]   (Linear weight is [out,in]; lib.rs:17162)
FTC_API void ftc_linear_f64(const double* x, const double* w, const double* b, double* y, int64_t m,
                            int64_t k, int64_t n) {
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      double s = 0.0;
      const double* xr = x + i * k;
      const double* wr = w + j * k;
      for (int64_t p = 0; p < k; ++p) s += xr[p] * wr[p];
      y[i * n + j] = s + (b ? b[j] : 0.0);
    }
}
// dx = dy.W ; dW = dy^T.x ; db = serial row sum   (lib.rs:17226)
FTC_API void ftc_linear_backward_f64(const double* x, const double* w, const double* dy, double* dx,
                                     double* dw, double* db, int64_t m, int64_t k, int64_t n) {
  if (dx)
    for (int64_t i = 0; i < m; ++i)
      for (int64_t p = 0; p < k; ++p) {
        double s = 0.0;
        for (int64_t j = 0; j < n; ++j) s += dy[i * n + j] * w[j * k + p];
        dx[i * k + p] = s;
      }
  if (dw)
    for (int64_t j = 0; j < n; ++j)
      for (int64_t p = 0; p < k; ++p) {
        double s = 0.0;
        for (int64_t i = 0; i < m; ++i) s += dy[i * n + j] * x[i * k + p];
        dw[j * k + p] = s;
      }
  if (db)
    for (int64_t j = 0; j < n; ++j) {
      double s = 0.0;
      for (int64_t i = 0; i < m; ++i) s += dy[i * n + j];
      db[j] = s;
    }
}
// Two-pass LayerNorm with population variance (lib.rs:5824)
FTC_API void ftc_layer_norm_f64(const double* x, const double* g, const double* b, double* y,
                                double* mean_out, double* rstd_out, int64_t rows, int64_t cols,
                                double eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const double* xr = x + r * cols;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += xr[c];
    const double mean = s / (double)cols;
    double q = 0.0;
    for (int64_t c = 0; c < cols; ++c) q += (xr[c] - mean) * (xr[c] - mean);
    const double rstd = 1.0 / std::sqrt(q / (double)cols + eps);
    for (int64_t c = 0; c < cols; ++c)
      y[r * cols + c] = (xr[c] - mean) * rstd * (g ? g[c] : 1.0) + (b ? b[c] : 0.0);
    if (mean_out) mean_out[r] = mean;
    if (rstd_out) rstd_out[r] = rstd;
  }
}
// Per-row cross entropy: lse - logit[target]; gradient g*(softmax - onehot)  (lib.rs:6649, :6679)
FTC_API void ftc_cross_entropy_f64(const double* logits, const int64_t* target, double* loss,
                                   double* dlogits, const double* gscale, int64_t rows,
                                   int64_t cols) {
  for (int64_t r = 0; r < rows; ++r) {
    const double* xr = logits + r * cols;
    double m = xr[0];
    for (int64_t c = 1; c < cols; ++c) m = std::max(m, xr[c]);
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += std::exp(xr[c] - m);
    const double lse = m + std::log(s);
    if (loss) loss[r] = lse - xr[target[r]];
    if (dlogits) {
      const double g = gscale ? gscale[r] : 1.0;
      for (int64_t c = 0; c < cols; ++c)
        dlogits[r * cols + c] = g * (std::exp(xr[c] - lse) - (c == target[r] ? 1.0 : 0.0));
    }
  }
}
// Scaled dot-product attention for one (batch*head): q,k,v [s,d]; causal masks j>i (lib.rs:4572)
FTC_API void ftc_sdpa_f64(const double* q, const double* k, const double* v, double* o, int64_t sq,
                          int64_t sk, int64_t d, double scale, int causal) {
  std::vector<double> p((size_t)sk);
  for (int64_t i = 0; i < sq; ++i) {
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
// AdamW single pass (ft-optim/src/lib.rs:1040-1054)
FTC_API void ftc_adamw_f64(double* p, const double* g, double* m, double* v, int64_t n, double lr,
                           double b1, double b2, double eps, double wd, int64_t step) {
  const double bc1 = 1.0 - std::pow(b1, (double)step), bc2 = 1.0 - std::pow(b2, (double)step);
  for (int64_t i = 0; i < n; ++i) {
    m[i] = b1 * m[i] + (1.0 - b1) * g[i];
    v[i] = b2 * v[i] + (1.0 - b2) * g[i] * g[i];
    const double mh = m[i] / bc1, vh = v[i] / bc2;
    p[i] -= p[i] * lr * wd + lr * mh / (std::sqrt(vh) + eps);
  }
}
// Metal-shader restatements (ft-kernel-metal/src/fused.rs:302 gelu, :321 softmax)
FTC_API void ftc_gelu_tanh_clamped_f32(const float* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    const float v = x[i];
    if (v >= 10.f) y[i] = v;
    else if (v <= -10.f) y[i] = 0.f;
    else y[i] = 0.5f * v * (1.f + std::tanh(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  }
}
FTC_API void ftc_softmax_guarded_f32(const float* x, float* y, int64_t rows, int64_t cols) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float m = -INFINITY;
    for (int64_t c = 0; c < cols; ++c) m = std::max(m, xr[c]);
    if (!std::isfinite(m)) {
      for (int64_t c = 0; c < cols; ++c) y[r * cols + c] = 0.f;
      continue;
    }
    float s = 0.f;
    for (int64_t c = 0; c < cols; ++c) s += std::exp(xr[c] - m);
    const float inv = s > 0.f ? 1.f / s : 0.f;
    for (int64_t c = 0; c < cols; ++c) y[r * cols + c] = std::exp(xr[c] - m) * inv;
  }
}
