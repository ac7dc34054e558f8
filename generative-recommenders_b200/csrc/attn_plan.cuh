// Work planning for the persistent tensor-core attention kernels.
//
// A tiny one-CTA kernel turns seq_offsets / num_targets into a list of (sequence, 128-row tile)
// work items ordered longest-first (counting sort on the number of opposite-side tiles an item
// has to visit).  Persistent CTAs then take items blockIdx.x, blockIdx.x + gridDim.x, ... so the
// expensive tiles of long sequences are spread over all SMs first and the cheap ones fill the
// tail.  The list lives in caller-provided scratch; nothing in it needs initialisation.
#pragma once

#include "common.cuh"

namespace b200hstu {

constexpr int TILE = 128;          // rows of a query tile == rows of a key/value tile
constexpr int PLAN_BUCKETS = 1024; // cost buckets of the counting sort
constexpr int PLAN_THREADS = 1024;

struct PlanHeader {
  int num_items;   // number of (sequence, tile) items
  int status;      // 0 = ok, else the site id of the first bounded wait that gave up
  int pad[2];
};

struct AttnGeomParams {
  const int32_t *seq_offsets, *num_targets;
  int B, H, max_seq_len, W, c, F;
};

struct TileItem {
  int b, mt;              // sequence, tile index inside the sequence
  int start, len, nt;     // first token row, untruncated length, number of targets
  int m0;                 // first row of the tile inside the sequence
  SeqMask m;
  int t_lo, n_main;       // opposite-side tiles [t_lo, t_lo + n_main)
  int extra_tile;         // >= 0: one more tile outside the main range (target rows' own diagonal)
  int n_tiles;
  int u;                  // first target position
  bool regular;           // tile classification shortcuts are valid
  __host__ __device__ __forceinline__ int tile_at(int j) const { return j < n_main ? t_lo + j : extra_tile; }
};

// kv tiles that the query tile `mt` of sequence `b` visits
__host__ __device__ __forceinline__ void fill_q_item(TileItem &it, const AttnGeomParams &g, int b, int mt, int start,
                                                     int len, int nt) {
  it.b = b;
  it.mt = mt;
  it.start = start;
  it.len = len;
  it.nt = nt;
  it.m0 = mt * TILE;
  it.m = make_seq_mask(it.len, g.max_seq_len, it.nt, g.c, g.W, g.F);
  it.u = it.len - it.nt;
  it.regular = (it.u >= g.c + 1) && (it.nt >= 0) && (it.len <= it.m.L);
  KvRange r = kv_range_for_q_tile(it.m, it.len, it.nt, it.m0, TILE);
  it.t_lo = r.lo / TILE;
  int t_hi = (r.hi + TILE - 1) / TILE;
  if (t_hi <= it.t_lo) t_hi = it.t_lo + 1;
  it.n_main = t_hi - it.t_lo;
  it.extra_tile = -1;
  if (r.diag_lo >= 0) {
    int dt = r.diag_lo / TILE;
    if (dt >= t_hi || dt < it.t_lo) it.extra_tile = dt;
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

// q tiles that the kv tile `nt_` of a sequence has to visit (backward, kv-stationary): a
// conservative contiguous range [t_lo, t_hi) plus, when contextual rows exist, tile 0.
__host__ __device__ __forceinline__ void fill_kv_item(TileItem &it, const AttnGeomParams &g, int b, int kt, int start,
                                                      int len, int nt) {
  it.b = b;
  it.mt = kt;
  it.start = start;
  it.len = len;
  it.nt = nt;
  it.m0 = kt * TILE;
  it.m = make_seq_mask(it.len, g.max_seq_len, it.nt, g.c, g.W, g.F);
  it.u = it.len - it.nt;
  it.regular = (it.u >= g.c + 1) && (it.nt >= 0) && (it.len <= it.m.L);
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
    if (g.c > 0 && kt > 0) it.extra_tile = 0;  // contextual rows (tile 0) see every non-target column
  }
  it.t_lo = t_lo;
  it.n_main = t_hi - t_lo;
  if (it.n_main < 0) it.n_main = 0;
  it.n_tiles = it.n_main + (it.extra_tile >= 0 ? 1 : 0);
}

template <bool KV_STATIONARY>
__global__ void __launch_bounds__(PLAN_THREADS) attn_plan_kernel(AttnGeomParams g, PlanHeader *hdr, int2 *items,
                                                                 int max_items) {
  __shared__ int hist[PLAN_BUCKETS];
  __shared__ int total;
  for (int i = threadIdx.x; i < PLAN_BUCKETS; i += PLAN_THREADS) hist[i] = 0;
  if (threadIdx.x == 0) total = 0;
  __syncthreads();
  for (int pass = 0; pass < 2; ++pass) {
    for (int b = threadIdx.x; b < g.B; b += PLAN_THREADS) {
      int len = g.seq_offsets[b + 1] - g.seq_offsets[b];
      int L = len < g.max_seq_len ? len : g.max_seq_len;
      int ntiles = (L + TILE - 1) / TILE;
      for (int t = 0; t < ntiles; ++t) {
        TileItem it;
        int nt = g.num_targets ? g.num_targets[b] : 0;
        if (KV_STATIONARY)
          fill_kv_item(it, g, b, t, 0, len, nt);
        else
          fill_q_item(it, g, b, t, 0, len, nt);
        int cost = it.n_tiles < PLAN_BUCKETS - 1 ? it.n_tiles : PLAN_BUCKETS - 1;
        int bucket = PLAN_BUCKETS - 1 - cost;  // expensive first
        if (pass == 0) {
          atomicAdd(&hist[bucket], 1);
        } else {
          int pos = atomicAdd(&hist[bucket], 1);
          if (pos < max_items) items[pos] = make_int2(b, t);
        }
      }
    }
    __syncthreads();
    if (pass == 0) {
      // exclusive prefix sum over the buckets (single thread: 1024 adds)
      if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < PLAN_BUCKETS; ++i) {
          int c = hist[i];
          hist[i] = run;
          run += c;
        }
        total = run;
      }
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) {
    hdr->num_items = total < max_items ? total : max_items;
    hdr->status = 0;
    hdr->pad[0] = hdr->pad[1] = 0;
  }
}

// device-side convenience: read the sequence geometry, then fill
template <bool KV_STATIONARY>
__device__ __forceinline__ void load_item(TileItem &it, const AttnGeomParams &g, int b, int t) {
  int start = g.seq_offsets[b];
  int len = g.seq_offsets[b + 1] - start;
  int nt = g.num_targets ? g.num_targets[b] : 0;
  if (KV_STATIONARY)
    fill_kv_item(it, g, b, t, start, len, nt);
  else
    fill_q_item(it, g, b, t, start, len, nt);
}

inline int64_t plan_max_items(int64_t total_L, int B) { return total_L / TILE + B + 1; }
inline int64_t plan_bytes(int64_t total_L, int B) {
  return (int64_t)sizeof(PlanHeader) + plan_max_items(total_L, B) * (int64_t)sizeof(int2);
}

}  // namespace b200hstu
