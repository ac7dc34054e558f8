// Work planning and tile geometry for the persistent tensor-core attention kernels.
//
// A tiny one-CTA kernel turns seq_offsets / num_targets into a list of work items ordered
// longest-first (counting sort on the number of opposite-side tiles an item has to visit).  Each
// item is a self-contained 32-byte descriptor (sequence, tile, first row, length, targets), so a
// persistent CTA needs one load per item and can fetch the next descriptor while it works on the
// current one.  Persistent CTAs take items blockIdx.x, blockIdx.x + gridDim.x, ... which spreads
// the expensive tiles of long sequences over all SMs first and lets the cheap ones fill the tail.
// The list lives in caller-provided scratch; nothing in it needs initialisation.
//
// Item kinds:
//   PLAN_Q_PAIR  forward: two consecutive 128-row query tiles of one sequence (they share K/V)
//   PLAN_Q_TILE  backward dQ: one 128-row query tile
//   PLAN_KV_TILE backward dK/dV: one 128-row key/value tile
#pragma once

#include "common.cuh"

namespace b200hstu {

constexpr int TILE = 128;          // rows of a query tile == rows of a key/value tile
constexpr int PLAN_BUCKETS = 1024; // cost buckets of the counting sort
constexpr int PLAN_THREADS = 1024;

enum PlanKind { PLAN_Q_PAIR = 0, PLAN_Q_TILE = 1, PLAN_KV_TILE = 2 };

struct PlanHeader {
  int num_items;   // number of work items (to be multiplied by the number of heads)
  int status;      // 0 = ok, else the site id of the first bounded wait that gave up
  int next;        // dynamic scheduling: next unclaimed (item, head) index; starts at the grid size
  int pad;
};

struct __align__(16) ItemDesc {
  int b, t;            // sequence, tile (or tile-pair) index inside the sequence
  int start, len, nt;  // first token row, untruncated length, number of targets
  int pad[3];
};

struct AttnGeomParams {
  const int32_t *seq_offsets, *num_targets;
  int B, H, max_seq_len, W, c, F;
  int delta;   // > 0: the query rows are the last `delta` positions of each sequence (cached inference)
};

// number of 128-row query tiles of a sequence and the position of the first query row
__host__ __device__ __forceinline__ int q_tiles_of(const AttnGeomParams &g, int L) {
  return ((g.delta > 0 ? g.delta : L) + 127) / 128;
}

struct TileItem {
  int b, mt;              // sequence, tile index inside the sequence
  int start, len, nt;     // first token row, untruncated length, number of targets
  int m0;                 // first row of the tile inside the sequence
  SeqMask m;
  int t_lo, n_main;       // opposite-side tiles [t_lo, t_lo + n_main)
  int extra_tile;         // >= 0: one more tile outside the main range
  int n_tiles;
  int u;                  // first target position
  bool regular;           // closed-form row intervals / tile classification are valid
  __host__ __device__ __forceinline__ int tile_at(int j) const { return j < n_main ? t_lo + j : extra_tile; }
  __host__ __device__ __forceinline__ bool visits(int t) const {
    return (t >= t_lo && t < t_lo + n_main) || t == extra_tile;
  }
};

__host__ __device__ __forceinline__ void fill_common(TileItem &it, const AttnGeomParams &g, int b, int t, int start,
                                                     int len, int nt) {
  it.b = b;
  it.mt = t;
  it.start = start;
  it.len = len;
  it.nt = nt;
  it.m = make_seq_mask(len, g.max_seq_len, nt, g.c, g.W, g.F);
  it.m0 = t * TILE + (g.delta > 0 ? it.m.L - g.delta : 0);
  it.u = len - nt;
  it.regular = (it.u >= g.c + 1) && (nt >= 0) && (len <= it.m.L);
}

// kv tiles that the query tile `mt` of a sequence visits
__host__ __device__ __forceinline__ void fill_q_item(TileItem &it, const AttnGeomParams &g, int b, int mt, int start,
                                                     int len, int nt) {
  fill_common(it, g, b, mt, start, len, nt);
  KvRange r = kv_range_for_q_tile(it.m, it.len, it.nt, it.m0, TILE);
  it.t_lo = r.lo / TILE;
  int t_hi = (r.hi + TILE - 1) / TILE;
  if (t_hi <= it.t_lo) t_hi = it.t_lo + 1;
  it.n_main = t_hi - it.t_lo;
  it.extra_tile = -1;
  if (r.diag_lo >= 0) {
    const int dt = r.diag_lo / TILE;
    const int d_end = r.diag_lo + TILE < it.m.L ? r.diag_lo + TILE : it.m.L;
    const int dt2 = (d_end - 1) / TILE;
    if (dt2 == dt) {
      if (dt >= t_hi || dt < it.t_lo) it.extra_tile = dt;
    } else {
      // a query tile that is not aligned to the kv tiles (cached inference): its diagonal block
      // straddles two kv tiles; widen the main range over both (tiles in between are masked out)
      if (dt2 + 1 > t_hi) t_hi = dt2 + 1;
      it.n_main = t_hi - it.t_lo;
    }
  }
  it.n_tiles = it.n_main + (it.extra_tile >= 0 ? 1 : 0);
}

// True when every (row, col) of the tile pair (rows of tile at m0, cols [n0, n0+TILE)) with
// row < L is valid, so the element-wise mask can be skipped.
__host__ __device__ __forceinline__ bool tile_pair_is_full(const TileItem &it, int n0) {
  if (!it.regular) return false;
  const SeqMask &m = it.m;
  if (it.m0 < m.c) return false;
  if (m.c > 0 && n0 < m.c) return false;
  int lim = it.m0 < it.u ? it.m0 : it.u;
  if (n0 + TILE > lim) return false;
  if (m.W > 0) {
    if (m.F > 0) return false;
    int rows_end = it.m0 + TILE < m.L ? it.m0 + TILE : m.L;
    int eff_last = rows_end - 1 < it.u ? rows_end - 1 : it.u;
    if (eff_last - n0 > m.W) return false;
  }
  return true;
}

// The kv tiles t for which tile_pair_is_full(it, t * TILE) holds form one range [lo, hi)
// (possibly empty): every condition above is a lower or an upper bound on n0.
struct FullRange {
  int lo, hi;
};
__host__ __device__ __forceinline__ FullRange full_tile_range(const TileItem &it) {
  FullRange r = {0, 0};
  if (!it.regular) return r;
  const SeqMask &m = it.m;
  if (it.m0 < m.c) return r;
  const int lim = it.m0 < it.u ? it.m0 : it.u;
  int lo = m.c > 0 ? (m.c + TILE - 1) / TILE : 0;
  if (m.W > 0) {
    if (m.F > 0) return r;
    const int rows_end = it.m0 + TILE < m.L ? it.m0 + TILE : m.L;
    const int eff_last = rows_end - 1 < it.u ? rows_end - 1 : it.u;
    const int first = eff_last - m.W;   // n0 >= first
    if (first > 0) {
      const int t = (first + TILE - 1) / TILE;
      lo = t > lo ? t : lo;
    }
  }
  r.lo = lo;
  r.hi = lim > 0 ? lim / TILE : 0;      // (t + 1) * TILE <= lim
  if (r.hi < r.lo) r.hi = r.lo;
  return r;
}

// q tiles that the kv tile `kt` of a sequence has to visit (backward, kv-stationary): a
// conservative contiguous range [t_lo, t_hi) plus, when contextual rows exist and fit one tile,
// tile 0.
__host__ __device__ __forceinline__ void fill_kv_item(TileItem &it, const AttnGeomParams &g, int b, int kt, int start,
                                                      int len, int nt) {
  fill_common(it, g, b, kt, start, len, nt);
  const int L = it.m.L;
  const int ntiles = (L + TILE - 1) / TILE;
  int t_lo = kt, t_hi = ntiles;
  it.extra_tile = -1;
  if (!it.regular) {
    t_lo = 0;
  } else {
    const int n0 = it.m0, n1 = it.m0 + TILE < L ? it.m0 + TILE : L;
    if (n0 >= it.u) {
      // only target columns: each is seen by its own row alone
      t_hi = kt + 1;
    } else if (g.W > 0 && g.F == 0) {
      // history rows i see j >= i - W; target rows see j >= u - W.  Last history row that can
      // still see a column of this tile: n1 - 1 + W.
      int last_row = n1 - 1 + g.W;
      bool targets_see = (it.u - (n1 - 1)) <= g.W || (g.c > 0 && n0 < g.c && it.u - g.c + 1 <= g.W);
      if (g.c > 0 && n0 < g.c) {
        // contextual columns are visible to rows with i - c + 1 <= W as well
        int lr = g.c - 1 + g.W;
        if (lr > last_row) last_row = lr;
      }
      if (!targets_see && it.nt > 0) {
        int hist_end = it.u - 1 < last_row ? it.u - 1 : last_row;
        t_hi = hist_end / TILE + 1;
      } else if (it.nt == 0) {
        int hist_end = L - 1 < last_row ? L - 1 : last_row;
        t_hi = hist_end / TILE + 1;
      }
      if (t_hi < kt + 1) t_hi = kt + 1;
      if (t_hi > ntiles) t_hi = ntiles;
    }
    if (g.c > 0 && n0 < it.u) {
      // contextual rows see every non-target column.  They sit in query tile 0 when the prefix
      // fits one tile; a longer prefix occupies several tiles, and the walk then starts at the
      // first tile (the element-wise mask clears the rows in between)
      if (g.c <= TILE) {
        if (kt > 0) it.extra_tile = 0;
      } else {
        t_lo = 0;
      }
    }
  }
  it.t_lo = t_lo;
  it.n_main = t_hi - t_lo;
  if (it.n_main < 0) it.n_main = 0;
  it.n_tiles = it.n_main + (it.extra_tile >= 0 ? 1 : 0);
}

// ---------------------------------------------------------------------------------------
// Two consecutive query tiles A (2p) and B (2p+1) that walk the union of their kv tiles
// ---------------------------------------------------------------------------------------
struct PairItem {
  TileItem A, B;
  bool hasB;
  int t_lo, n_main;
  int extra0, extra1;   // up to two tiles outside the main range (target rows' own diagonal blocks)
  int n_extra;
  int n_tiles;
  __host__ __device__ __forceinline__ int tile_at(int j) const {
    return j < n_main ? t_lo + j : (j == n_main ? extra0 : extra1);
  }
};

__host__ __device__ __forceinline__ void fill_pair_item(PairItem &p, const AttnGeomParams &g, int b, int pair,
                                                        int start, int len, int nt) {
  // With an odd number of query tiles the tile left without a partner is the FIRST one (a single
  // kv tile), not the last and most expensive one: a query tile on its own cannot overlap its
  // score products with its activation and runs ~1.6x longer per kv tile.
  const int L = len < g.max_seq_len ? len : g.max_seq_len;
  const int ntiles = q_tiles_of(g, L);
  const bool odd = (ntiles & 1) != 0;
  const int first = odd ? (pair == 0 ? 0 : 2 * pair - 1) : 2 * pair;
  fill_q_item(p.A, g, b, first, start, len, nt);
  p.hasB = !(odd && pair == 0) && (first + 1) < ntiles;
  int lo = p.A.t_lo, hi = p.A.t_lo + p.A.n_main;
  if (p.hasB) {
    fill_q_item(p.B, g, b, first + 1, start, len, nt);
    lo = p.B.t_lo < lo ? p.B.t_lo : lo;
    int bh = p.B.t_lo + p.B.n_main;
    hi = bh > hi ? bh : hi;
  } else {
    p.B = p.A;
    p.B.n_main = 0;
    p.B.extra_tile = -1;
    p.B.n_tiles = 0;
  }
  p.t_lo = lo;
  p.n_main = hi - lo;
  p.n_extra = 0;
  p.extra0 = p.extra1 = -1;
  int ea = p.A.extra_tile, eb = p.hasB ? p.B.extra_tile : -1;
  if (ea >= 0 && (ea < lo || ea >= hi)) {
    p.extra0 = ea;
    p.n_extra = 1;
  }
  if (eb >= 0 && (eb < lo || eb >= hi) && eb != ea) {
    if (p.n_extra == 0) p.extra0 = eb; else p.extra1 = eb;
    ++p.n_extra;
  }
  p.n_tiles = p.n_main + p.n_extra;
}

// ---------------------------------------------------------------------------------------
// Closed-form mask of one query row on the regular domain: the valid columns of row i are
//   [lo, hi)  united with  [0, ctx_hi)  united with  {i}
// (history window, contextual prefix, self).  Equals SeqMask::valid() for every column < L.
// ---------------------------------------------------------------------------------------
struct RowInterval {
  int lo, hi, ctx_hi, self;
};

__host__ __device__ __forceinline__ RowInterval row_interval(const TileItem &it, int i) {
  RowInterval r;
  const int c = it.m.c, W = it.m.W, F = it.m.F, u = it.u;
  r.self = i;
  if (i < c) {  // contextual row: everything before the targets
    r.lo = 0;
    r.hi = u;
    r.ctx_hi = 0;
    return r;
  }
  const bool tgt = i >= u;
  const int eff = tgt ? u : i;
  const bool full = (W == 0) || (F > 0 && (tgt || i >= u - F));
  r.hi = tgt ? u : i + 1;
  int lo = full ? c : eff - W;
  r.lo = lo < c ? c : lo;
  const bool ctx_ok = full || (eff - c + 1 <= W);
  r.ctx_hi = ctx_ok ? (c < r.hi ? c : r.hi) : 0;
  return r;
}

__host__ __device__ __forceinline__ uint32_t low_bits(int n) {  // n clamped to [0, 32] -> n low bits set
  n = n < 0 ? 0 : n;
  return n >= 32 ? 0xffffffffu : ((1u << n) - 1u);
}

// validity bits of columns base .. base+31 for the row described by r (columns >= L are cleared)
__host__ __device__ __forceinline__ uint32_t row_mask_bits(const RowInterval &r, int base, int L) {
  uint32_t bits = low_bits(r.hi - base) & ~low_bits(r.lo - base);
  bits |= low_bits(r.ctx_hi - base);
  int d = r.self - base;
  if (d >= 0 && d < 32) bits |= 1u << d;
  return bits & low_bits(L - base);
}

// The transposed view for the K/V-stationary backward: the valid query rows of key column j are
//   [a1, b1)  u  [a2, b2)  u  [0, c3)  u  [a4, L)  u  {j}
// (history rows inside the window, history rows of the full-attention tail, contextual rows,
// target rows).  Equals SeqMask::valid(i, j) for every row < L on the regular domain.
struct ColInterval {
  int a1, b1, a2, b2, c3, a4, self;
};

__host__ __device__ __forceinline__ ColInterval col_interval(const TileItem &it, int j) {
  ColInterval r;
  const int c = it.m.c, W = it.m.W, F = it.m.F, u = it.u, L = it.m.L;
  r.self = j;
  r.a1 = r.b1 = r.a2 = r.b2 = 0;
  r.c3 = 0;
  r.a4 = L;
  if (j >= u) return r;  // a target column is seen by its own row only
  const int jc = j > c - 1 ? j : c - 1;  // contextual columns behave like position c - 1 for the window
  int lo1 = jc + 1 > c ? jc + 1 : c;
  r.a1 = lo1;
  r.b1 = (W == 0) ? u : (jc + W + 1 < u ? jc + W + 1 : u);
  if (W > 0 && F > 0) {
    r.a2 = lo1 > u - F ? lo1 : u - F;
    r.b2 = u;
  }
  r.c3 = c;
  if (W == 0 || F > 0 || u - jc <= W) r.a4 = u;
  return r;
}

__host__ __device__ __forceinline__ uint32_t range_bits(int a, int b, int base) {
  return low_bits(b - base) & ~low_bits(a - base);
}

// validity bits of query rows base .. base+31 for the key column described by r
__host__ __device__ __forceinline__ uint32_t col_mask_bits(const ColInterval &r, int base, int L) {
  uint32_t bits = range_bits(r.a1, r.b1, base) | range_bits(r.a2, r.b2, base) | low_bits(r.c3 - base) |
                  range_bits(r.a4, L, base);
  int d = r.self - base;
  if (d >= 0 && d < 32) bits |= 1u << d;
  return bits & low_bits(L - base);
}

template <int KIND>
__host__ __device__ __forceinline__ int item_cost(const AttnGeomParams &g, int b, int t, int len, int nt) {
  if (KIND == PLAN_Q_PAIR) {
    PairItem p;
    fill_pair_item(p, g, b, t, 0, len, nt);
    // a query tile without a partner takes about 1.6x as long per kv tile
    return p.hasB ? p.A.n_tiles + p.B.n_tiles : (p.A.n_tiles * 8 + 4) / 5;
  } else if (KIND == PLAN_Q_TILE) {
    TileItem it;
    fill_q_item(it, g, b, t, 0, len, nt);
    return it.n_tiles;
  } else {
    TileItem it;
    fill_kv_item(it, g, b, t, 0, len, nt);
    return it.n_tiles;
  }
}

template <int KIND>
__device__ __forceinline__ void plan_body(const AttnGeomParams &g, PlanHeader *hdr, ItemDesc *items, int max_items,
                                          int first_dynamic) {
  static_assert(PLAN_BUCKETS == PLAN_THREADS, "one bucket per thread in the scan");
  __shared__ int hist[PLAN_BUCKETS];
  __shared__ int warp_sums[32];
  __shared__ int total;
  for (int i = threadIdx.x; i < PLAN_BUCKETS; i += PLAN_THREADS) hist[i] = 0;
  if (threadIdx.x == 0) total = 0;
  __syncthreads();
  // threads are laid out as 64 sequences x 16 tile slots so that the (sequence, tile) pairs of a
  // batch are costed in parallel instead of one thread walking all tiles of a sequence
  constexpr int TSLOTS = 16;
  constexpr int BSLOTS = PLAN_THREADS / TSLOTS;
  const int tslot = threadIdx.x % TSLOTS, bslot = threadIdx.x / TSLOTS;
  // the cost of the first item a thread meets is kept for the second pass (batches of up to 64
  // sequences of up to 16 units give every thread at most one item)
  int kept_bucket = -1;
  for (int pass = 0; pass < 2; ++pass) {
    bool first = true;
    for (int b = bslot; b < g.B; b += BSLOTS) {
      const int start = g.seq_offsets[b];
      const int len = g.seq_offsets[b + 1] - start;
      const int nt = g.num_targets ? g.num_targets[b] : 0;
      const int L = len < g.max_seq_len ? len : g.max_seq_len;
      const int ntiles = KIND == PLAN_KV_TILE ? (L + TILE - 1) / TILE : q_tiles_of(g, L);
      const int nunits = KIND == PLAN_Q_PAIR ? (ntiles + 1) / 2 : ntiles;
      for (int t = tslot; t < nunits; t += TSLOTS) {
        int bucket;
        if (first && pass == 1 && kept_bucket >= 0) {
          bucket = kept_bucket;
        } else {
          int cost = item_cost<KIND>(g, b, t, len, nt);
          cost = cost < PLAN_BUCKETS - 1 ? cost : PLAN_BUCKETS - 1;
          bucket = PLAN_BUCKETS - 1 - cost;  // expensive first
          if (first && pass == 0) kept_bucket = bucket;
        }
        first = false;
        if (pass == 0) {
          atomicAdd(&hist[bucket], 1);
        } else {
          int pos = atomicAdd(&hist[bucket], 1);
          if (pos < max_items) {
            ItemDesc d;
            d.b = b; d.t = t; d.start = start; d.len = len; d.nt = nt;
            d.pad[0] = d.pad[1] = d.pad[2] = 0;
            items[pos] = d;
          }
        }
      }
    }
    __syncthreads();
    if (pass == 0) {
      // exclusive prefix sum over the buckets: one bucket per thread, warp scans + scan of warp sums
      const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
      const int mine = hist[threadIdx.x];
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (lane == 31) warp_sums[wid] = incl;
      __syncthreads();
      if (wid == 0) {
        int ws = warp_sums[lane];
        int wincl = ws;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int v = __shfl_up_sync(0xffffffffu, wincl, o);
          if (lane >= o) wincl += v;
        }
        warp_sums[lane] = wincl - ws;  // exclusive offset of each warp
        if (lane == 31) total = wincl;
      }
      __syncthreads();
      hist[threadIdx.x] = warp_sums[wid] + incl - mine;
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) {
    hdr->num_items = total < max_items ? total : max_items;
    hdr->status = 0;
    hdr->next = first_dynamic;
    hdr->pad = 0;
  }
}

// ---------------------------------------------------------------------------------------
// Relative position bias as the kernels read it: a table over the signed distance i - j,
//   ext[k] = bias[|k|] / 2  for |k| < numel, else 0,   k in (-P, P),
// so that a thread walking along a row (or a column) reads consecutive entries with constant
// offsets from one pointer: no absolute value, no bounds test, no index arithmetic per element.
// (The factor 1/2 is the h = x / 2 of the tanh form of SiLU.)  The table lives at the start of
// the caller's scratch and is rebuilt by the planning launch of every call that has a bias.
//
// P covers every distance a thread can form, not only those of valid pairs: rows and columns of a
// tile beyond the end of a sequence (up to the next multiple of 128, plus the second query tile of
// a forward pair that does not exist, plus the offset of an unaligned query tile of the cached-
// inference forward) are read before they are masked, so P = roundup128(N) + 256.
// ---------------------------------------------------------------------------------------
struct BiasTable {
  const float *src;   // bias_by_distance [numel]; NULL = no bias
  int numel;
  float *dst;         // 2 P - 1 floats
  int N;              // max_seq_len
  __host__ __device__ __forceinline__ int half_width() const { return (N + 127) / 128 * 128 + 256; }
  // the entry of distance 0
  __host__ __device__ __forceinline__ const float *centre() const { return dst + (half_width() - 1); }
};
inline int64_t bias_table_bytes(const void *bias, int max_seq_len) {
  if (bias == nullptr) return 0;
  const int64_t P = ((int64_t)max_seq_len + 127) / 128 * 128 + 256;
  int64_t n = (2 * P - 1) * (int64_t)sizeof(float);
  return (n + 255) / 256 * 256;
}
__device__ __forceinline__ void build_bias_table(const BiasTable &t) {
  if (t.src == nullptr) return;
  const int P = t.half_width();
  for (int x = threadIdx.x; x < 2 * P - 1; x += blockDim.x) {
    const int k = x - (P - 1);
    const int a = k < 0 ? -k : k;
    t.dst[x] = a < t.numel ? 0.5f * t.src[a] : 0.f;
  }
}

template <int KIND>
__global__ void __launch_bounds__(PLAN_THREADS) attn_plan_kernel(AttnGeomParams g, PlanHeader *hdr, ItemDesc *items,
                                                                 int max_items, int first_dynamic, BiasTable bt) {
  build_bias_table(bt);
  // the attention kernel that follows may already set itself up; it waits for this grid to
  // finish before it reads the list
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  plan_body<KIND>(g, hdr, items, max_items, first_dynamic);
}

// two work lists in one launch (one CTA each): the backward's K/V-tile and query-tile lists
template <int KIND0, int KIND1>
__global__ void __launch_bounds__(PLAN_THREADS) attn_plan2_kernel(AttnGeomParams g, PlanHeader *hdr0, ItemDesc *items0,
                                                                  PlanHeader *hdr1, ItemDesc *items1, int max_items,
                                                                  int first_dynamic, BiasTable bt) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (blockIdx.x == 0) build_bias_table(bt);
  if (blockIdx.x == 0)
    plan_body<KIND0>(g, hdr0, items0, max_items, first_dynamic);
  else
    plan_body<KIND1>(g, hdr1, items1, max_items, first_dynamic);
}

// all three work lists of a training step in one launch (one CTA each): forward, then the
// backward's K/V-tile and query-tile lists
template <int KIND0>
__global__ void __launch_bounds__(PLAN_THREADS) attn_plan3_kernel(AttnGeomParams g, PlanHeader *hdr0, ItemDesc *items0,
                                                                  PlanHeader *hdr1, ItemDesc *items1, PlanHeader *hdr2,
                                                                  ItemDesc *items2, int max_items, int first_dynamic,
                                                                  BiasTable bt) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (blockIdx.x == 0) build_bias_table(bt);
  if (blockIdx.x == 0)
    plan_body<KIND0>(g, hdr0, items0, max_items, first_dynamic);
  else if (blockIdx.x == 1)
    plan_body<PLAN_KV_TILE>(g, hdr1, items1, max_items, first_dynamic);
  else
    plan_body<PLAN_Q_TILE>(g, hdr2, items2, max_items, first_dynamic);
}

__device__ __forceinline__ ItemDesc load_desc(const ItemDesc *items, int idx) {
  const int4 *p4 = reinterpret_cast<const int4 *>(items + idx);
  int4 a = __ldg(p4), b = __ldg(p4 + 1);
  ItemDesc d;
  d.b = a.x; d.t = a.y; d.start = a.z; d.len = a.w; d.nt = b.x;
  d.pad[0] = d.pad[1] = d.pad[2] = 0;
  return d;
}

// ---------------------------------------------------------------------------------------
// Dynamic work distribution inside a persistent CTA.
//
// Every CTA starts with the (item, head) index blockIdx.x and claims further indices from the
// counter in the plan header with atomicAdd, so CTAs that drew cheap items simply take more of
// them.  One thread (the TMA producer) claims the index, reads the item's descriptor and publishes
// both through a small shared-memory ring guarded by mbarriers; the MMA warp and the activation
// warps pick them up from there (no global-memory latency on their critical path).  An index at or
// beyond the total ends the loop of every role.
// ---------------------------------------------------------------------------------------
constexpr int SCHED_SLOTS = 4;
constexpr int SCHED_SLOT_BYTES = 32;
constexpr int SCHED_CONSUMERS = 9;  // MMA warp + 8 activation warps, one arrival each

struct SchedMsg {
  ItemDesc d;
  int idx;
};

inline int64_t plan_max_items(int64_t total_L, int B) { return total_L / TILE + B + 1; }
inline int64_t plan_bytes(int64_t total_L, int B) {
  int64_t n = (int64_t)sizeof(PlanHeader) + plan_max_items(total_L, B) * (int64_t)sizeof(ItemDesc);
  return (n + 255) / 256 * 256;
}

}  // namespace b200hstu
