// Device side of the sm_100a bf16 GEMM: TMA -> 128B-swizzled smem ring -> tcgen05.mma (fp32
// accumulators in TMEM, double buffered) -> tcgen05.ld epilogue, as one persistent kernel.
//
// The same kernel carries three collective-fused forms (template parameter COMM = 1), in
// which the last `comm_ctas` CTAs of the grid move data over NVLink while the others compute:
//   gather A / gather B : the row-sharded operand is pulled shard by shard from the peers
//                         (bulk async copies peer -> smem -> local staging buffer, no cluster
//                         multicast), a flag per 128-row subtile is published, and the TMA
//                         producer of a compute CTA waits only for the subtiles its tile reads.
//                         Tiles are visited own-shard-first in rank-rotated order.
//   scatter-reduce D    : the epilogue stores each partial tile as bf16 straight into the
//                         inbox of the rank that owns those rows (peer stores), then raises a
//                         flag at the owner; the comm CTAs of the owner add the partials of
//                         all ranks in ascending rank order and apply bias / residual /
//                         accumulate.  The order is fixed, so the sum is reproducible.
// Every wait on a flag that another CTA or rank sets is bounded and ends in the status word.
#pragma once
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

constexpr int G_BM = 128;
constexpr int G_BK = 64;
constexpr int G_UMMA_K = 16;
constexpr int G_EPI_WARPS = 8;
constexpr int G_THREADS = 64 + 32 * G_EPI_WARPS;
constexpr int G_MAX_RANKS = 8;
constexpr int G_COPY_SLOT = 32768;   // bytes per bulk copy of the gather ring
constexpr int G_COPY_SLOTS = 6;
constexpr int G_SCATTER_BATCH = 8;   // reduce-scatter tiles per system-scope fence
constexpr long long G_PEER_WAIT_CYCLES = 4000000000ll;

struct GemmArgs {
  int M, N, K, L0, L1;
  int a_mn, b_mn;
  void* D;
  long long ldd, d_s0, d_s1;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  long long ldr, r_s0, r_s1;
  __nv_bfloat16* aux;  // optional bf16 copy of the pre-activation (same layout as D)
  float alpha;
  int epi;
  int out_fp32;
  int accumulate;
  int splits;          // >1: split-K, partial tiles go to `ws` as fp32 [split][M][N]
  float* ws;
  int* status;
  // Ragged rows (expert batches): the M rows of batch l are segments of `seg_rows` rows of which
  // only the first seg_counts[l * segs + s] are in use; a 128-row tile without a used row is
  // skipped by every role (no loads, no MMAs, no stores).  NULL = all rows in use.
  const int* seg_counts;
  int seg_rows;
};

// True when rows [m_t * 128, m_t * 128 + 128) of batch l hold at least one row in use.  Every role of a
// CTA evaluates this for the same items, so the pipelines stay in step.
__device__ __forceinline__ bool tile_has_rows(const GemmArgs& p, int l, int m_t) {
  if (!p.seg_counts) return true;
  const int row0 = m_t * 128, row1 = min(p.M, row0 + 128);
  const int segs = (p.M + p.seg_rows - 1) / p.seg_rows;
  for (int sg = row0 / p.seg_rows; sg <= (row1 - 1) / p.seg_rows; ++sg) {
    const int lo = sg * p.seg_rows, hi = lo + __ldg(p.seg_counts + l * segs + sg);
    if (max(row0, lo) < min(row1, hi)) return true;
  }
  return false;
}

struct CommArgs {
  int mode;                      // FTK_COMM_*
  int rank, world, comm_ctas;
  int chunk_rows;                // rows of the sharded operand / output owned by one rank
  long long sub_bytes;           // bytes of one 128-row subtile of the gathered operand
  const uint8_t* src[G_MAX_RANKS];   // gather: shard of rank r, contiguous [chunk_rows, K]
  uint8_t* full;                 // gather: local staging of the whole operand
  int* sub_flags;                // gather: one word per 128-row subtile, holds the epoch
  int* ready_local;              // gather: [world] words written by the peers (may be null)
  int* ready_peer[G_MAX_RANKS];  // gather: word `rank` of peer r's ready_local
  int push;                      // gather: 1 = every rank stores its own shard into the peers' staging
  uint8_t* full_peer[G_MAX_RANKS];   // push gather: staging buffer of rank r (entry `rank` == full)
  int* flags_peer[G_MAX_RANKS];      // push gather: sub_flags of rank r (entry `rank` == sub_flags)
  __nv_bfloat16* inbox[G_MAX_RANKS];  // scatter: inbox of rank r, [world][chunk_rows][N]
  int* arrive[G_MAX_RANKS];      // scatter: flags of rank r, [tiles of one chunk][world]
  const int* epoch;              // device word: use count (>= 1) of the flag arrays
};

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = G_BM * G_BK * 2;
  static constexpr int B_BYTES = BN * G_BK * 2;
  static constexpr int STAGES = (BN == 128) ? 6 : 4;
  static constexpr int ACC_STRIDE = (BN == 192) ? 256 : BN;  // TMEM columns between accumulators
  static constexpr int TMEM_COLS = (BN == 128) ? 256 : 512;  // power of two
  static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/ +
                              G_EPI_WARPS * 4096 /*output staging tiles*/;
};

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Epilogue activations use the hardware tanh (relative error ~2^-11, below bf16 rounding).
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanh_fast(u));
}
__device__ __forceinline__ float gelu_tanh_grad_fast(float x) {
  const float x2 = x * x;
  const float t = tanh_fast(0.7978845608028654f * (x + 0.044715f * x * x2));
  const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

// v[i] = f(v[i], rr[i]) for the 32 values of one row chunk; the switch is outside the loop.
__device__ __forceinline__ void apply_epi32(float* v, const float* rr, int epi) {
  switch (epi) {
    case FTK_EPI_GELU_TANH:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
      break;
    case FTK_EPI_GELU_ERF:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_erf_f(v[i]);
      break;
    case FTK_EPI_RELU:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = v[i] > 0.f ? v[i] : 0.f;
      break;
    case FTK_EPI_MUL_DGELU_TANH:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= gelu_tanh_grad_fast(rr[i]);
      break;
    case FTK_EPI_MUL_DGELU_ERF:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= gelu_erf_grad_f(rr[i]);
      break;
    case FTK_EPI_MUL_DRELU:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = rr[i] > 0.f ? v[i] : 0.f;
      break;
    default:
      break;
  }
}

// ------------------------------------------------------------------ coalescing bf16 output stores
// One warp's staging tile: 32 rows x 128 B in shared memory, 16-byte segments XOR-swizzled by
// the row.  A thread `put`s the packed bf16 of its row for one 32-column chunk; after two chunks
// (or at the end of the tile) `flush` reads the tile transposed so that 8 consecutive lanes
// write 128 contiguous bytes (4 lanes / 64 bytes when only one chunk is staged) of one row.
struct OutStager {
  uint8_t* tile;
  __nv_bfloat16* d_base;       // row 0 of the output (of this batch entry)
  long long row0, ldd;         // first output row of this warp's slab, leading dimension
  int M, lane, staged, n_start;
  bool usable;
  __device__ __forceinline__ OutStager(uint8_t* t, const GemmArgs& p, __nv_bfloat16* d, long long r0, int ln)
      : tile(t), d_base(d), row0(r0), ldd(p.ldd), M(p.M), lane(ln), staged(0), n_start(0) {
    usable = !p.out_fp32 && !p.accumulate && p.splits == 1 && (p.ldd % 8 == 0) &&
             ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
  }
  __device__ __forceinline__ void put(const float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 o;
      o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
      o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
      o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
      o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
      *reinterpret_cast<uint4*>(tile + lane * 128 + (((staged * 4 + i) ^ (lane & 7)) << 4)) = o;
    }
  }
  __device__ __forceinline__ void chunk_done(int n0) {
    if (staged == 0) n_start = n0;
    if (++staged == 2) flush();
  }
  __device__ __forceinline__ void flush() {
    if (staged == 0) return;
    __syncwarp();
    if (staged == 2) {
      const int seg = lane & 7;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3);
        const uint4 o = *reinterpret_cast<const uint4*>(tile + rr * 128 + ((seg ^ (rr & 7)) << 4));
        if (row0 + rr < M) *reinterpret_cast<uint4*>(d_base + (row0 + rr) * ldd + n_start + seg * 8) = o;
      }
    } else {
      const int seg = lane & 3;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rr = 8 * i + (lane >> 2);
        const uint4 o = *reinterpret_cast<const uint4*>(tile + rr * 128 + ((seg ^ (rr & 7)) << 4));
        if (row0 + rr < M) *reinterpret_cast<uint4*>(d_base + (row0 + rr) * ldd + n_start + seg * 8) = o;
      }
    }
    __syncwarp();
    staged = 0;
  }
};

// ------------------------------------------------------------------ flags between CTAs / ranks
__device__ __forceinline__ int ld_acq_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acq_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_rel_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_rel_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
// Bounded wait until *p >= want.  SYS selects system scope (flags written by another GPU).
template <bool SYS>
__device__ __forceinline__ bool flag_wait(const int* p, int want, const WaitCtx& c) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  while ((SYS ? ld_acq_sys(p) : ld_acq_gpu(p)) < want) {
    __nanosleep(64);
    if ((++spins & 31u) == 0u) {
      if (aborted(c)) return false;
      if (clock64() - t0 > G_PEER_WAIT_CYCLES) {
        raise_abort(c, FT_ERR_WAIT_PEER);
        return false;
      }
    }
  }
  return true;
}

// Bulk async copies without cluster multicast: global (local or peer) -> this CTA's smem, and
// smem -> local global memory.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Work item -> output tile.  Plain GEMMs walk m fastest; the collective forms walk the row
// chunks of the sharded dimension in rank-rotated order.
struct TileCoord {
  int sp, l, m_t, n_t;
};
template <int BN, int COMM>
__device__ __forceinline__ TileCoord decode_item(int item, const GemmArgs& p, const CommArgs& c,
                                                 int tiles_m, int tiles_n, int nbatch) {
  TileCoord t;
  if (!COMM || c.mode == FTK_COMM_NONE || (c.mode == FTK_COMM_GATHER_B && p.b_mn)) {
    const int tiles_mn = tiles_m * tiles_n;
    t.sp = item / (tiles_mn * nbatch);
    const int rem = item - t.sp * (tiles_mn * nbatch);
    t.l = rem / tiles_mn;
    const int tt = rem - t.l * tiles_mn;
    t.m_t = tt % tiles_m;
    t.n_t = tt / tiles_m;
    return t;
  }
  t.sp = 0;
  t.l = 0;
  if (c.mode == FTK_COMM_GATHER_B) {
    const int shift = (int)(((long long)c.rank * c.chunk_rows) / BN);
    t.n_t = (item / tiles_m + shift) % tiles_n;
    t.m_t = item % tiles_m;
  } else {  // row chunks of A (gather) or D (scatter): own chunk first / last
    const int tpc = c.chunk_rows / G_BM;
    const int per_chunk = tpc * tiles_n;
    const int i = item / per_chunk;
    const int rem = item - i * per_chunk;
    const int chunk = (c.rank + i + (c.mode == FTK_COMM_SCATTER_D ? 1 : 0)) % c.world;
    t.n_t = rem / tpc;
    t.m_t = chunk * tpc + rem % tpc;
  }
  return t;
}

// ------------------------------------------------------------------ comm CTAs: gather
// The gathered operand is cut into pieces of at most G_COPY_SLOT bytes.  Pieces are visited in
// rank-rotated order and dealt round robin to the comm CTAs, so the data of the first tiles is
// fetched by many CTAs at once.  In each comm CTA one thread drives an smem ring: bulk loads
// (from the peer's shard, or from this rank's own shard) run four pieces ahead of the bulk
// stores into the local staging buffer; a flag word per piece is published once its store has
// landed.  With `own_aside` (activation gathers) the ring moves the remote chunks only: the GEMM
// reads own-shard tiles straight from the shard (second tensor map), and the staged copy of the
// own chunk, which only serves later consumers of the gathered operand, is made by the other
// warps of the copy CTAs with plain 16-byte loads and stores while the ring runs.
//
// Push form (c.push): the roles of the two sides are exchanged.  Every rank stores its OWN shard
// into every rank's staging buffer and publishes the piece's flag AT THE CONSUMER with a
// system-scope release, so that consumers only ever poll their own memory.  The loader thread
// fills the ring from local memory with bulk loads; one storer warp per slot drains it with plain
// 16-byte peer stores, which are posted and so are not bound by NVLink round trips the way peer
// loads are (bulk stores to a peer were measured at a quarter of the rate of these).  The work list is destination-major in the order the
// consumers need their chunks: rank P's data is the first remote chunk of rank P-1, the second of
// P-2, ...; at any time each GPU sends one chunk to one peer and receives one chunk from one peer
// at the full link rate, and a consumer's next chunk is complete after 1/(W-1) of the exchange.
// The copy into this rank's own staging buffer comes first for weight gathers (tiles that
// straddle two chunks wait for its flags) and last for activation gathers (the GEMM reads own
// tiles from the shard; the staged copy only serves later kernels).  The caller alternates two
// staging buffers between consecutive calls: a rank can be at most one collective ahead of a
// peer, so the buffer it writes is never the one that peer still reads.
__device__ __forceinline__ void comm_gather(uint8_t* smem, uint64_t* bars, const CommArgs& c,
                                            int epoch, int cta, bool own_last, const WaitCtx& ctx) {
  uint64_t* full = bars;
  // progress word shared by the storer (thread 64) and the publisher (thread 32): number of this
  // CTA's pieces whose stores have landed; -1 after a failure
  int* progress = reinterpret_cast<int*>(bars + 2 * G_COPY_SLOTS);
  const int spc = c.chunk_rows / G_BM;                 // subtiles per chunk
  const uint32_t piece = c.sub_bytes < G_COPY_SLOT ? (uint32_t)c.sub_bytes : (uint32_t)G_COPY_SLOT;
  const int pps = (int)(c.sub_bytes / piece);          // pieces per subtile
  const int ppc = spc * pps;                           // pieces per chunk
  const bool push = c.push != 0;
  const bool own_aside = own_last && !push;
  // pieces are numbered by distance from this rank: [0, ppc) is the own chunk (pull), or by
  // destination in the order the consumers need them (push)
  const int first = own_aside ? ppc : 0;
  const int n_pieces = ppc * c.world - first;
  const int mine = cta < n_pieces ? (n_pieces - cta + c.comm_ctas - 1) / c.comm_ctas : 0;
  auto rotated = [&](int i) { return first + (int)(((long long)cta + (long long)i * c.comm_ctas) % n_pieces); };
  // piece number -> the rank whose memory is read (pull) / written (push)
  auto other = [&](int q) {
    const int dd = q / ppc;
    if (!push) return (c.rank + dd) % c.world;
    if (own_last) return dd == c.world - 1 ? c.rank : (c.rank - 1 - dd + 2 * c.world) % c.world;
    return (c.rank - dd + c.world) % c.world;
  };
  if (own_aside && threadIdx.x >= 96) {
    // own chunk: shard -> its place in the gathered operand, 8 vectors in flight per thread
    const long long nvec = (long long)ppc * piece / 16;
    const uint4* src = reinterpret_cast<const uint4*>(c.src[c.rank]);
    uint4* dst = reinterpret_cast<uint4*>(c.full + (long long)c.rank * ppc * piece);
    const long long nthr = (long long)c.comm_ctas * (blockDim.x - 96);
    const long long t0 = (long long)cta * (blockDim.x - 96) + (threadIdx.x - 96);
    for (long long v0 = t0; v0 < nvec; v0 += 8 * nthr) {
      uint4 u[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const long long v = v0 + k * nthr;
        if (v < nvec) u[k] = __ldg(src + v);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const long long v = v0 + k * nthr;
        if (v < nvec) dst[v] = u[k];
      }
    }
    return;
  }
  uint64_t* empty = bars + G_COPY_SLOTS;
  if (push && threadIdx.x >= 96) {
    // push form, storer warps: one warp per ring slot (a warp that served several slots could meet a
    // slot's barrier a whole phase early and take its parity for "complete").  Warp sw copies the pieces
    // i = sw, sw + slots, ... from slot sw to the consumer's staging buffer with 16-byte peer stores
    // (posted: no round trip), frees the slot and publishes the piece's flag at the consumer.
    const int lane = threadIdx.x & 31, sw = (int)(threadIdx.x >> 5) - 3;
    static_assert(G_THREADS / 32 - 3 >= G_COPY_SLOTS, "one storer warp per ring slot");
    if (sw >= G_COPY_SLOTS) return;
    const int nv = (int)(piece >> 4);
    // A system-scope fence waits until the peer has acknowledged every store of the thread (microseconds
    // over NVLink), so a slot is freed as soon as its bytes are in registers / on their way, and the
    // flags of PUSH_BATCH pieces are published behind one fence.
    constexpr int PUSH_BATCH = 4;
    int* pend[PUSH_BATCH];
    int n_pend = 0;
    for (int i = sw; i < mine; i += G_COPY_SLOTS) {
      const int slot = sw;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&full[slot], (uint32_t)((i / G_COPY_SLOTS) & 1), ctx, FT_ERR_WAIT_FULL) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      __syncwarp();
      if (!ok) return;
      const int q = rotated(i);
      const int dest = other(q);
      const uint4* s4 = reinterpret_cast<const uint4*>(smem + slot * G_COPY_SLOT);
      uint4* d4 = reinterpret_cast<uint4*>(c.full_peer[dest] + ((long long)c.rank * ppc + q % ppc) * piece);
#pragma unroll 8
      for (int v = lane; v < nv; v += 32) d4[v] = s4[v];
      __syncwarp();                                   // every lane has read its part of the slot
      if (lane == 0) mbar_arrive(&empty[slot]);
      pend[n_pend++] = c.flags_peer[dest] + c.rank * ppc + q % ppc;
      if (n_pend == PUSH_BATCH || i + G_COPY_SLOTS >= mine) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0)
          for (int k = 0; k < n_pend; ++k) st_rel_sys(pend[k], epoch);
        n_pend = 0;
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    // loader: peer (or own) memory -> ring slot.  It never waits for a store to land, only for
    // the slot's previous contents to have been read out, so up to G_COPY_SLOTS loads are in
    // flight per CTA.
    if (cta == 0 && c.ready_local) {
      // announce that this rank's shard is final for this epoch
      __threadfence_system();
      for (int r = 0; r < c.world; ++r)
        if (r != c.rank) st_rel_sys(c.ready_peer[r], epoch);
    }
    int ready_seen = 1 << c.rank;
    for (int i = 0; i < mine; ++i) {
      const int slot = i % G_COPY_SLOTS;
      if (i >= G_COPY_SLOTS &&
          !mbar_wait(&empty[slot], (uint32_t)(((i / G_COPY_SLOTS) - 1) & 1), ctx, FT_ERR_WAIT_EMPTY))
        break;
      const int q = rotated(i);
      const int chunk = push ? c.rank : other(q);
      if (c.ready_local && !((ready_seen >> chunk) & 1)) {
        if (!flag_wait<true>(c.ready_local + chunk, epoch, ctx)) break;
        ready_seen |= 1 << chunk;
      }
      mbar_arrive_expect_tx(&full[slot], piece);
      bulk_load(smem + slot * G_COPY_SLOT, c.src[chunk] + (long long)(q % ppc) * piece, piece, &full[slot]);
    }
  } else if (!push && threadIdx.x == 64) {
    // storer: ring slot -> the gathered operand in this GPU's memory; frees a slot once its store
    // has read it and advances the progress word once stores have landed
    int stored = 0;
    bool ok = true;
    while (stored < mine) {
      const int slot = stored % G_COPY_SLOTS;
      if (!mbar_wait(&full[slot], (uint32_t)((stored / G_COPY_SLOTS) & 1), ctx, FT_ERR_WAIT_FULL)) {
        ok = false;
        break;
      }
      const int q = rotated(stored);
      bulk_store(c.full + ((long long)other(q) * ppc + q % ppc) * piece, smem + slot * G_COPY_SLOT, piece);
      bulk_wait_group_read<1>();                       // the previous store has read its slot
      if (stored > 0) mbar_arrive(&empty[(stored - 1) % G_COPY_SLOTS]);
      ++stored;
      bulk_wait_group<3>();                            // all but the newest three stores landed
      if (stored > 3) asm volatile("st.release.cta.shared.s32 [%0], %1;" ::"r"(smem_u32(progress)), "r"(stored - 3) : "memory");
    }
    bulk_wait_group<0>();
    asm volatile("st.release.cta.shared.s32 [%0], %1;" ::"r"(smem_u32(progress)), "r"(ok ? stored : -1) : "memory");
  } else if (!push && threadIdx.x == 32) {
    // publisher: turns the driver's progress into per-piece flags.  It owns no copies in flight,
    // so its release stores never wait behind the ring.
    int published = 0;
    const long long t0 = clock64();
    while (published < mine) {
      int done;
      asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(done) : "r"(smem_u32(progress)) : "memory");
      if (done < 0) return;
      if (done == published) {
        __nanosleep(100);
        if (clock64() - t0 > 2 * G_PEER_WAIT_CYCLES) return;   // the driver's own waits are bounded
        continue;
      }
      for (; published < done; ++published) {
        const int q = rotated(published);
        st_rel_gpu(c.sub_flags + other(q) * ppc + q % ppc, epoch);
      }
    }
  }
}

// ------------------------------------------------------------------ ordered reduce
// Tile (n_t, m_in) of this rank's chunk: out = sum over source ranks (ascending) of the bf16
// partials in the local inbox, + bias, + residual, (+ previous output).  Run by `nthr` threads
// of a CTA (thread index `tid`), which synchronise on the abort-aware warp barrier `wbar` (one
// arrival per participating warp); tiles are dealt round robin over `n_ctas` CTAs.  Every compute CTA calls this after its last GEMM tile, so the
// whole GPU's bandwidth drains the inbox.
template <int BN>
__device__ __forceinline__ void comm_reduce(const GemmArgs& p, const CommArgs& c, int epoch, int cta,
                                            int n_ctas, int tid, int nthr, const WaitCtx& ctx,
                                            uint64_t* wbar, uint32_t& wbar_ph) {
  const int tpc = c.chunk_rows / G_BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int n_tiles = tpc * tiles_n;
  const __nv_bfloat16* inbox = c.inbox[c.rank];
  const long long src_stride = (long long)c.chunk_rows * p.N;
  constexpr int U = 4;                                  // vectors in flight per thread and source
  for (int t = cta; t < n_tiles; t += n_ctas) {
    if (tid < c.world) flag_wait<true>(c.arrive[c.rank] + t * c.world + tid, epoch, ctx);
    if (!warps_barrier(wbar, wbar_ph, tid & 31, ctx) || aborted(ctx)) return;
    const int n_t = t / tpc, m_in = t % tpc;
    const int n_base = n_t * BN;
    const int cols = min(BN, p.N - n_base);            // multiple of 8
    const int vec_per_row = cols >> 3;
    const int n_vec = G_BM * vec_per_row;
    for (int v0 = tid; v0 < n_vec; v0 += nthr * U) {
      float acc[U][8];
      long long off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * nthr;
        const int row = m_in * G_BM + v / vec_per_row;  // row inside this rank's chunk
        const int col = n_base + ((v % vec_per_row) << 3);
        off[u] = v < n_vec ? (long long)row * p.N + col : -1;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
      }
#pragma unroll 2
      for (int s = 0; s < c.world; ++s) {
        uint4 w[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          w[u] = off[u] >= 0 ? __ldcg(reinterpret_cast<const uint4*>(inbox + s * src_stride + off[u]))
                             : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float2 f0 = unpack_bf16(w[u].x), f1 = unpack_bf16(w[u].y), f2 = unpack_bf16(w[u].z),
                       f3 = unpack_bf16(w[u].w);
          acc[u][0] += f0.x; acc[u][1] += f0.y; acc[u][2] += f1.x; acc[u][3] += f1.y;
          acc[u][4] += f2.x; acc[u][5] += f2.y; acc[u][6] += f3.x; acc[u][7] += f3.y;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (off[u] < 0) continue;
        const int v = v0 + u * nthr;
        const int row = m_in * G_BM + v / vec_per_row;
        const int col = n_base + ((v % vec_per_row) << 3);
        float* a8 = acc[u];
        if (p.bias) {
#pragma unroll
          for (int i = 0; i < 8; ++i) a8[i] += __bfloat162float(__ldg(p.bias + col + i));
        }
        if (p.resid) {
          const uint4 r4 = *reinterpret_cast<const uint4*>(p.resid + (long long)row * p.ldr + col);
          const float2 f0 = unpack_bf16(r4.x), f1 = unpack_bf16(r4.y), f2 = unpack_bf16(r4.z),
                       f3 = unpack_bf16(r4.w);
          a8[0] += f0.x; a8[1] += f0.y; a8[2] += f1.x; a8[3] += f1.y;
          a8[4] += f2.x; a8[5] += f2.y; a8[6] += f3.x; a8[7] += f3.y;
        }
        if (p.out_fp32) {
          float* dp = reinterpret_cast<float*>(p.D) + (long long)row * p.ldd + col;
          float4 x = make_float4(a8[0], a8[1], a8[2], a8[3]);
          float4 y = make_float4(a8[4], a8[5], a8[6], a8[7]);
          if (p.accumulate) {
            const float4 ox = reinterpret_cast<float4*>(dp)[0], oy = reinterpret_cast<float4*>(dp)[1];
            x.x += ox.x; x.y += ox.y; x.z += ox.z; x.w += ox.w;
            y.x += oy.x; y.y += oy.y; y.z += oy.z; y.w += oy.w;
          }
          reinterpret_cast<float4*>(dp)[0] = x;
          reinterpret_cast<float4*>(dp)[1] = y;
        } else {
          __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)row * p.ldd + col;
          if (p.accumulate) {
            const uint4 o4 = *reinterpret_cast<const uint4*>(dp);
            const float2 f0 = unpack_bf16(o4.x), f1 = unpack_bf16(o4.y), f2 = unpack_bf16(o4.z),
                         f3 = unpack_bf16(o4.w);
            a8[0] += f0.x; a8[1] += f0.y; a8[2] += f1.x; a8[3] += f1.y;
            a8[4] += f2.x; a8[5] += f2.y; a8[6] += f3.x; a8[7] += f3.y;
          }
          uint4 o;
          o.x = pack_bf16(a8[0], a8[1]);
          o.y = pack_bf16(a8[2], a8[3]);
          o.z = pack_bf16(a8[4], a8[5]);
          o.w = pack_bf16(a8[6], a8[7]);
          *reinterpret_cast<uint4*>(dp) = o;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ gather, pushed by the epilogue warps
// Third form of the gather (c.push == 3): no CTA is set aside for copying.  The eight epilogue warps of EVERY
// CTA spend most of a tile's main loop waiting for the accumulator; in that time they store this rank's shard
// into the peers' staging buffers, 4 KB per poll of the accumulator barrier, so all 148 SMs issue peer stores
// (a single SM sustains 8 - 17 GB/s over NVLink, the link needs many of them) and none is taken from the
// product.  Pieces are numbered destination-major in the order the consumers need them and dealt round robin
// to the (CTA, warp) pairs; a warp publishes the flags of up to four finished pieces behind one system fence.
// Pushing never waits for anything, and a warp with pieces left never blocks on its accumulator without
// pushing, so every shard is delivered whatever the peers' tiles are waiting for.
struct EpiPusher {
  const CommArgs& c;
  int lane, ppc, n_total, stride, nv, own_last;
  uint32_t piece;
  int pj;          // piece this warp is working on (>= n_total: done)
  int pv;          // vectors of it already stored
  int* pend[4];
  int n_pend;
  int batch;       // finished pieces whose flags go out behind one fence

  __device__ __forceinline__ EpiPusher(const CommArgs& c_, bool active, int gw, int n_warps, int lane_,
                                       bool own_last_)
      : c(c_), lane(lane_), own_last(own_last_ ? 1 : 0), pv(0), n_pend(0) {
    if (!active) {        // not a pushing launch: nothing to do, nothing of `c` is looked at
      ppc = n_total = stride = nv = batch = 0;
      piece = 0;
      pj = 1;
      return;
    }
    const int spc = c.chunk_rows / G_BM;
    piece = c.sub_bytes < G_COPY_SLOT ? (uint32_t)c.sub_bytes : (uint32_t)G_COPY_SLOT;
    ppc = spc * (int)(c.sub_bytes / piece);
    n_total = ppc * c.world;
    stride = n_warps;
    nv = (int)(piece >> 4);
    pj = gw;
    // a warp with few pieces publishes each at once (a consumer waits for it), one with many amortises the fence
    const int per_warp = (n_total + n_warps - 1) / n_warps;
    batch = per_warp >= 16 ? 4 : (per_warp >= 8 ? 2 : 1);
  }
  __device__ __forceinline__ bool busy() const { return pj < n_total; }
  __device__ __forceinline__ int dest_of(int d) const {
    if (own_last) return d == c.world - 1 ? c.rank : (c.rank - 1 - d + 2 * c.world) % c.world;
    return (c.rank - d + c.world) % c.world;
  }
  __device__ __forceinline__ void publish() {
    if (n_pend == 0) return;
    __threadfence_system();
    __syncwarp();
    if (lane == 0)
      for (int k = 0; k < n_pend; ++k) st_rel_sys(pend[k], *c.epoch);
    __syncwarp();
    n_pend = 0;
  }
  // stores the next 4 KB (8 vectors per lane) of the current piece
  __device__ __forceinline__ void step() {
    if (pj >= n_total) return;
    const int d = pj / ppc, q = pj - d * ppc;
    const int dest = dest_of(d);
    const uint4* src = reinterpret_cast<const uint4*>(c.src[c.rank] + (long long)q * piece);
    uint4* dst = reinterpret_cast<uint4*>(c.full_peer[dest] + ((long long)c.rank * ppc + q) * piece);
    uint4 u[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int v = pv + k * 32 + lane;
      if (v < nv) u[k] = __ldg(src + v);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int v = pv + k * 32 + lane;
      if (v < nv) dst[v] = u[k];
    }
    pv += 256;
    if (pv >= nv) {
      pend[n_pend++] = c.flags_peer[dest] + c.rank * ppc + q;
      pv = 0;
      pj += stride;
      if (n_pend >= batch || pj >= n_total) publish();
    }
  }
};

// ------------------------------------------------------------------ the kernel
template <int BN, int COMM>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_bf16_sm100_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmOwn, const GemmArgs p, const CommArgs c) {
  using Cfg = GemmCfg<BN>;
  static_assert(!COMM || G_COPY_SLOTS * G_COPY_SLOT <= Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES),
                "gather ring must fit the operand ring");
  static_assert(!COMM || 2 * G_COPY_SLOTS <= 2 * Cfg::STAGES + 4, "barrier space");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + Cfg::STAGES * Cfg::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES));
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::STAGES;
  uint64_t* tfull = bars + 2 * Cfg::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);
  uint64_t* wbar = tempty + 3;            // barrier among the epilogue warps (all warps of a reduce CTA)
  static_assert((2 * Cfg::STAGES + 6) * 8 <= 256, "barrier space");
  uint32_t wbar_ph = 0;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};

  const int n_compute = COMM ? (int)gridDim.x - c.comm_ctas : (int)gridDim.x;
  const bool comm_cta = COMM && (int)blockIdx.x >= n_compute;
  const int epoch = COMM ? *c.epoch : 0;

  if (threadIdx.x == 0) {
    if (comm_cta) {
      for (int i = 0; i < G_COPY_SLOTS; ++i) {
        mbar_init(&bars[i], 1);
        mbar_init(&bars[G_COPY_SLOTS + i], 1);
      }
      *reinterpret_cast<int*>(bars + 2 * G_COPY_SLOTS) = 0;   // gather progress word
    } else {
      for (int i = 0; i < Cfg::STAGES; ++i) {
        mbar_init(&full[i], 1);
        mbar_init(&empty[i], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&tfull[i], 1);
        mbar_init(&tempty[i], G_EPI_WARPS);
      }
    }
    mbar_init(wbar, comm_cta ? G_THREADS / 32 : G_EPI_WARPS);
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == 1 && !comm_cta) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (comm_cta) {
    if (COMM) {
      const int cta = (int)blockIdx.x - n_compute;
      if (c.mode == FTK_COMM_SCATTER_D)
        comm_reduce<BN>(p, c, epoch, (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x, G_THREADS, ctx, wbar,
                        wbar_ph);
      else
        comm_gather(smem, bars, c, epoch, cta,
                    /*own_last=*/c.mode == FTK_COMM_GATHER_A, ctx);
    }
    __syncthreads();
    return;
  }
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + G_BM - 1) / G_BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_mn = tiles_m * tiles_n;
  const int nbatch = p.L0 * p.L1;
  const int total = tiles_mn * nbatch * p.splits;  // work item = (split, batch, n tile, m tile)
  const int kblocks_all = (p.K + G_BK - 1) / G_BK;
  const int kb_per_split = (kblocks_all + p.splits - 1) / p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
    }
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    int k_ready = 0;
    // flag words per 128-row subtile of a gathered operand (one per copied piece)
    const int pps = !COMM ? 1 : (c.sub_bytes > G_COPY_SLOT ? (int)(c.sub_bytes / G_COPY_SLOT) : 1);
    // (An L2 prefetch cursor running 8 k-blocks ahead of the ring was measured and removed: the
    // extra TMA requests slowed the mainloop by 1.7x.)
    for (int item = blockIdx.x; ok && item < total; item += n_compute) {
      const TileCoord t = decode_item<BN, COMM>(item, p, c, tiles_m, tiles_n, nbatch);
      if (!tile_has_rows(p, t.l, t.m_t)) continue;
      const int m_t = t.m_t, n_t = t.n_t;
      const int l0 = t.l % p.L0, l1 = t.l / p.L0;
      const int kb0 = t.sp * kb_per_split;
      const int kb1 = min(kblocks_all, kb0 + kb_per_split);
      const bool k_sharded = COMM && c.mode == FTK_COMM_GATHER_B && p.b_mn;
      // operand tiles that lie wholly inside this rank's own shard are read from the shard itself
      const CUtensorMap* mapA = &tmA;
      const CUtensorMap* mapB = &tmB;
      int a_row = m_t * G_BM, b_row = n_t * BN;
      bool own = false;
      if (COMM && !k_sharded && c.mode == FTK_COMM_GATHER_A) {
        own = (a_row / c.chunk_rows == c.rank);
        if (own) {
          mapA = &tmOwn;
          a_row -= c.rank * c.chunk_rows;
        }
      } else if (COMM && !k_sharded && c.mode == FTK_COMM_GATHER_B) {
        own = c.chunk_rows >= BN && b_row >= c.rank * c.chunk_rows &&
              min(p.N, b_row + BN) <= (c.rank + 1) * c.chunk_rows;
        if (own) {
          mapB = &tmOwn;
          b_row -= c.rank * c.chunk_rows;
        }
      }
      if (COMM && !k_sharded && !own && (c.mode == FTK_COMM_GATHER_A || c.mode == FTK_COMM_GATHER_B)) {
        // the staged subtiles this tile reads must have landed
        int f0, f1;
        if (c.mode == FTK_COMM_GATHER_A) {
          f0 = f1 = m_t;
        } else {
          f0 = (n_t * BN) / G_BM;
          f1 = (min(p.N, n_t * BN + BN) - 1) / G_BM;
        }
        // one flag per piece; the lanes poll the pieces of subtiles f0..f1 in parallel
        int good = 1;
        for (int pc = f0 * pps + lane; pc < (f1 + 1) * pps && good; pc += 32)
          good = (c.push ? flag_wait<true>(c.sub_flags + pc, epoch, ctx)
                         : flag_wait<false>(c.sub_flags + pc, epoch, ctx)) ? 1 : 0;
        fence_proxy_async_all();
        if (!__all_sync(0xffffffffu, good)) break;
      }
      for (int kb = kb0; kb < kb1; ++kb) {
        if (k_sharded) {
          // B is sharded along K: rows [0, k_ready * 128) of the staged operand are known final
          const int need = (min(p.K, kb * G_BK + G_BK) - 1) / G_BM + 1;
          while (ok && k_ready < need) {
            int good = 1;
            for (int pc = k_ready * pps + lane; pc < (k_ready + 1) * pps && good; pc += 32)
              good = (c.push ? flag_wait<true>(c.sub_flags + pc, epoch, ctx)
                             : flag_wait<false>(c.sub_flags + pc, epoch, ctx)) ? 1 : 0;
            fence_proxy_async_all();
            if (!__all_sync(0xffffffffu, good)) ok = false;
            ++k_ready;
          }
          if (!ok) break;
        }
        if (!mbar_wait(&empty[s], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES);
          uint8_t* a_dst = sA + s * Cfg::A_BYTES;
          uint8_t* b_dst = sB + s * Cfg::B_BYTES;
          if (!p.a_mn) {
            tma_load_4d(a_dst, mapA, &full[s], kb * G_BK, a_row, l0, l1);
          } else {
#pragma unroll
            for (int cc = 0; cc < G_BM / 64; ++cc)
              tma_load_4d(a_dst + cc * (G_BK * 128), &tmA, &full[s], m_t * G_BM + cc * 64, kb * G_BK,
                          l0, l1);
          }
          if (!p.b_mn) {
            tma_load_4d(b_dst, mapB, &full[s], kb * G_BK, b_row, l0, l1);
          } else {
#pragma unroll
            for (int cc = 0; cc < BN / 64; ++cc)
              tma_load_4d(b_dst + cc * (G_BK * 128), &tmB, &full[s], n_t * BN + cc * 64, kb * G_BK,
                          l0, l1);
          }
        }
        __syncwarp();
        if (++s == Cfg::STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_bf16(G_BM, BN, p.a_mn, p.b_mn);
    const uint32_t a_lbo = p.a_mn ? G_BK * 128 : 16, a_adv = p.a_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
    const uint32_t b_lbo = p.b_mn ? G_BK * 128 : 16, b_adv = p.b_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
    const uint32_t a_lo0 = desc_lo(smem_u32(sA), a_lbo), b_lo0 = desc_lo(smem_u32(sB), b_lbo);
    const uint32_t a_adv16 = a_adv >> 4, b_adv16 = b_adv >> 4;
    int s = 0;
    uint32_t ph = 0;
    int acc = 0;
    uint32_t acc_ph = 0;  // bit a = phase of accumulator a
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total; item += n_compute) {
      if (p.seg_counts) {
        const TileCoord tc = decode_item<BN, COMM>(item, p, c, tiles_m, tiles_n, nbatch);
        if (!tile_has_rows(p, tc.l, tc.m_t)) continue;
      }
      const int sp = (COMM && c.mode != FTK_COMM_NONE) ? 0 : item / (tiles_mn * nbatch);
      const int kb0 = sp * kb_per_split;
      const int kb1 = min(kblocks_all, kb0 + kb_per_split);
      if (!mbar_wait(&tempty[acc], ((acc_ph >> acc) & 1u) ^ 1u, ctx, FT_ERR_WAIT_TMEM_EMPTY)) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full[s], ph, ctx, FT_ERR_WAIT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          // descriptor low words of this stage, stepped by (bytes >> 4) per k-step
          const uint32_t a_lo = a_lo0 + (uint32_t)s * (Cfg::A_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)s * (Cfg::B_BYTES >> 4);
          umma_bf16_lo(d_tmem, a_lo, b_lo, idesc, kb > kb0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < G_BK / G_UMMA_K; ++k)
            umma_bf16_lo(d_tmem, a_lo + k * a_adv16, b_lo + k * b_adv16, idesc, 1u);
          umma_commit(&empty[s]);
          if (kb == kb1 - 1) umma_commit(&tfull[acc]);
        }
        __syncwarp();
        if (++s == Cfg::STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (kb1 <= kb0 && lane == 0) umma_commit(&tfull[acc]);  // empty split: nothing to wait for
      __syncwarp();
      acc_ph ^= (1u << acc);
      acc ^= 1;
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps)
    const int ew = warp - 2;
    const int q = warp & 3;               // TMEM lane quarter this warp may read
    const int half = ew >> 2;             // which half of the tile's columns
    const int row_in_tile = q * 32 + lane;
    constexpr int CHUNKS = BN / 32;
    constexpr int C_HALF = (CHUNKS + 1) / 2;
    const int c_begin = half == 0 ? 0 : C_HALF;
    const int c_end = half == 0 ? C_HALF : CHUNKS;
    int acc = 0;
    uint32_t acc_ph = 0;
    int pend_owner[G_SCATTER_BATCH], pend_tile[G_SCATTER_BATCH], n_pend = 0;   // scatter: unpublished tiles
    bool epi_ok = true;   // false once this warp gave up a wait: it then skips every later barrier
    const bool ew_push = COMM && c.push == 3 && (c.mode == FTK_COMM_GATHER_A || c.mode == FTK_COMM_GATHER_B);
    EpiPusher pusher(c, ew_push, (int)blockIdx.x * G_EPI_WARPS + ew, n_compute * G_EPI_WARPS, lane,
                     c.mode == FTK_COMM_GATHER_A);
    for (int item = blockIdx.x; item < total; item += n_compute) {
      const TileCoord t = decode_item<BN, COMM>(item, p, c, tiles_m, tiles_n, nbatch);
      if (!tile_has_rows(p, t.l, t.m_t)) continue;
      const int sp = t.sp, l = t.l, m_t = t.m_t, n_t = t.n_t;
      const int l0 = l % p.L0, l1 = l / p.L0;
      const bool empty_split = (sp * kb_per_split >= kblocks_all);
      if (COMM && ew_push) {
        // push 4 KB of the shard per poll while the accumulator is not ready
        while (pusher.busy()) {
          int ready = (lane == 0 && mbar_try_wait(&tfull[acc], (acc_ph >> acc) & 1u)) ? 1 : 0;
          ready = __shfl_sync(0xffffffffu, ready, 0);
          if (ready || aborted(ctx)) break;
          pusher.step();
        }
      }
      if (!mbar_wait(&tfull[acc], (acc_ph >> acc) & 1u, ctx, FT_ERR_WAIT_TMEM_FULL)) {
        epi_ok = false;
        break;
      }
      tc_fence_after();
      const long long row = (long long)m_t * G_BM + row_in_tile;
      if (COMM && c.mode == FTK_COMM_SCATTER_D) {
        // partial tile -> inbox of the owning rank, slot of this rank; then one flag per tile
        const int tpc = c.chunk_rows / G_BM;
        const int owner = m_t / tpc;
        // first row of this warp's 32-row slab inside the owner's chunk, in this rank's inbox slot
        const long long slab_row = (long long)m_t * G_BM + q * 32 - (long long)owner * c.chunk_rows;
        __nv_bfloat16* ob = c.inbox[owner] + ((long long)c.rank * c.chunk_rows + slab_row) * p.N;
        // Peer stores want long contiguous runs: two 32-column chunks are packed to bf16,
        // transposed through a per-warp smem tile (32 rows x 128 B, XOR-swizzled 16-byte
        // segments) and written so that 8 consecutive lanes cover 128 contiguous bytes of a row.
        uint8_t* stage = smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES) + 256 + ew * 4096;
#pragma unroll 1
        for (int ci = c_begin; ci < c_end; ci += 2) {
          const int c0 = ci * 32;
          uint32_t r[64];
          tmem_ld32(tmem_base + acc * Cfg::ACC_STRIDE + c0 + ((uint32_t)(q * 32) << 16), r);
          tmem_ld32(tmem_base + acc * Cfg::ACC_STRIDE + c0 + 32 + ((uint32_t)(q * 32) << 16), r + 32);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[8 * j + 0]) * p.alpha, __uint_as_float(r[8 * j + 1]) * p.alpha);
            o.y = pack_bf16(__uint_as_float(r[8 * j + 2]) * p.alpha, __uint_as_float(r[8 * j + 3]) * p.alpha);
            o.z = pack_bf16(__uint_as_float(r[8 * j + 4]) * p.alpha, __uint_as_float(r[8 * j + 5]) * p.alpha);
            o.w = pack_bf16(__uint_as_float(r[8 * j + 6]) * p.alpha, __uint_as_float(r[8 * j + 7]) * p.alpha);
            *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
          }
          __syncwarp();
          const int n0 = n_t * BN + c0;
          const int seg = lane & 7;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 4 * i + (lane >> 3);
            const uint4 o = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((seg ^ (rr & 7)) << 4));
            if ((long long)m_t * G_BM + q * 32 + rr < p.M && n0 + seg * 8 < p.N)
              *reinterpret_cast<uint4*>(ob + (long long)rr * p.N + n0 + seg * 8) = o;
          }
          __syncwarp();
        }
        // the accumulator is drained: release it before waiting for the peer stores to land
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        // A system-scope fence waits for every peer store of this thread to be acknowledged
        // (tens of microseconds under load), so arrival flags are published in batches: one
        // fence per G_SCATTER_BATCH tiles instead of one per tile.
        pend_owner[n_pend] = owner;
        pend_tile[n_pend] = n_t * tpc + (m_t - owner * tpc);
        if (++n_pend == G_SCATTER_BATCH) {
          __threadfence_system();
          if (!warps_barrier(wbar, wbar_ph, lane, ctx)) {
            epi_ok = false;
            break;
          }
          if (ew == 0 && lane == 0)
            for (int i = 0; i < n_pend; ++i)
              st_rel_sys(c.arrive[pend_owner[i]] + pend_tile[i] * c.world + c.rank, epoch);
          n_pend = 0;
        }
        acc_ph ^= (1u << acc);
        acc ^= 1;
        continue;
      }
      const long long d_off = l0 * p.d_s0 + l1 * p.d_s1 + row * p.ldd;
      const long long r_off = l0 * p.r_s0 + l1 * p.r_s1 + row * p.ldr;
      const bool need_r = p.resid != nullptr;
      // bf16 outputs leave through a per-warp smem tile (32 rows x 128 B, XOR-swizzled 16-byte
      // segments): a thread owns one row of the accumulator, so direct stores would touch 32
      // rows per instruction with 16 bytes each; after the transpose 8 consecutive lanes write
      // 128 contiguous bytes of one row.
      OutStager stager(smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES) + 256 + ew * 4096, p,
                       reinterpret_cast<__nv_bfloat16*>(p.D) + l0 * p.d_s0 + l1 * p.d_s1,
                       (long long)m_t * G_BM + q * 32, lane);
#pragma unroll 1
      for (int ci = c_begin; ci < c_end; ++ci) {
        const int c0 = ci * 32;
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * Cfg::ACC_STRIDE + c0 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        const int n0 = n_t * BN + c0;
        const bool stage_this = stager.usable && n0 + 32 <= p.N;     // warp-uniform
        if (!stage_this) stager.flush();
        if (row < p.M && n0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = empty_split ? 0.f : __uint_as_float(r[i]) * p.alpha;
          const bool full_chunk = (n0 + 32 <= p.N);
          if (p.splits > 1) {
            // raw partial tile -> workspace [split][batch][M][N] (fp32)
            float* wp = p.ws + (((long long)sp * nbatch + l) * p.M + row) * p.N + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(wp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(wp)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N) wp[i] = v[i];
            }
            continue;
          }
          if (p.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (full_chunk || n0 + i < p.N) v[i] += __bfloat162float(__ldg(p.bias + n0 + i));
          }
          if (p.aux) {
            __nv_bfloat16* ap = p.aux + d_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(ap) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 o;
                o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
                o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
                o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
                reinterpret_cast<uint4*>(ap)[i] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N) ap[i] = __float2bfloat16(v[i]);
            }
          }
          float rr[32];
          if (need_r) {
            const __nv_bfloat16* rp = p.resid + r_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 u = __ldg(reinterpret_cast<const uint4*>(rp) + i);
                float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z),
                       f3 = unpack_bf16(u.w);
                rr[8 * i + 0] = f0.x; rr[8 * i + 1] = f0.y; rr[8 * i + 2] = f1.x;
                rr[8 * i + 3] = f1.y; rr[8 * i + 4] = f2.x; rr[8 * i + 5] = f2.y;
                rr[8 * i + 6] = f3.x; rr[8 * i + 7] = f3.y;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                rr[i] = (n0 + i < p.N) ? __bfloat162float(rp[i]) : 0.f;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = 0.f;
          }
          const bool r_is_operand = (p.epi >= FTK_EPI_MUL_DGELU_TANH);
          if (p.epi != FTK_EPI_NONE) apply_epi32(v, rr, p.epi);
          if (need_r && !r_is_operand) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += rr[i];
          }
          if (p.out_fp32) {
            float* dp = reinterpret_cast<float*>(p.D) + d_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                if (p.accumulate) {
                  float4 old = reinterpret_cast<float4*>(dp)[i];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                reinterpret_cast<float4*>(dp)[i] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N) dp[i] = p.accumulate ? dp[i] + v[i] : v[i];
            }
          } else if (stage_this) {
            stager.put(v);
          } else {
            __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + d_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (p.accumulate) {
                  uint4 u = reinterpret_cast<uint4*>(dp)[i];
                  float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z),
                         f3 = unpack_bf16(u.w);
                  v[8 * i + 0] += f0.x; v[8 * i + 1] += f0.y; v[8 * i + 2] += f1.x;
                  v[8 * i + 3] += f1.y; v[8 * i + 4] += f2.x; v[8 * i + 5] += f2.y;
                  v[8 * i + 6] += f3.x; v[8 * i + 7] += f3.y;
                }
                uint4 o;
                o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
                o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
                o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
                reinterpret_cast<uint4*>(dp)[i] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N)
                  dp[i] = __float2bfloat16(p.accumulate ? __bfloat162float(dp[i]) + v[i] : v[i]);
            }
          }
        }
        if (stage_this) stager.chunk_done(n0);     // every lane of the warp, also rows past M
      }
      stager.flush();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc_ph ^= (1u << acc);
      acc ^= 1;
    }
    if (COMM && ew_push) {
      // whatever of the shard is still here goes out now (also after an abort: the peers wait for it)
      while (pusher.busy()) pusher.step();
      pusher.publish();
    }
    // A warp that gave up a wait (epi_ok false) goes straight to the teardown: its siblings are
    // at, or will reach, a bounded warps_barrier and leave the same way once they see the abort flag.
    if (COMM && c.mode == FTK_COMM_SCATTER_D && epi_ok && n_pend > 0) {   // the last, partial batch of flags
      __threadfence_system();
      if (!warps_barrier(wbar, wbar_ph, lane, ctx)) epi_ok = false;
      if (epi_ok && ew == 0 && lane == 0)
        for (int i = 0; i < n_pend; ++i)
          st_rel_sys(c.arrive[pend_owner[i]] + pend_tile[i] * c.world + c.rank, epoch);
    }
    // reduce-scatter: with the GEMM tiles done, the epilogue warps of every CTA drain the inbox
    if (COMM && c.mode == FTK_COMM_SCATTER_D && epi_ok && !aborted(ctx))
      comm_reduce<BN>(p, c, epoch, (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x - 64,
                      32 * G_EPI_WARPS, ctx, wbar, wbar_ph);
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_f) {
    // give copies and MMAs still in flight time to land before smem/TMEM go away
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace ftk
