// Inclusive scan of a few very long rows in ONE pass over the data (8 bytes per element), with a result
// that does not depend on timing.
//
// The three-phase form (chunk totals, scan of the totals, scan with carry-in) reads the data twice:
// 12 bytes per element. A "decoupled look-back" scan reads it once, but which partial sums a tile
// finds published depends on timing, so its roundings are not reproducible. Here a tile (one warp,
// 2048 elements kept in registers) publishes only its own AGGREGATE, which depends on nothing else,
// and aggregates are combined along a fixed tree of fan-out 32: the warp that completes a group of 32
// (an atomic counter tells it) adds the group's 32 values in lane order and publishes the group's
// aggregate one level up, and so on. A tile's carry-in is then
//     (earlier groups at the top level) + ... + (earlier groups at level 1) + (earlier tiles of its group),
// each a fixed-order sum of at most 31 published values: the same bits whatever the timing. Nothing
// published depends on a carry, so there is no chain of waits: a tile only waits until the tiles before
// it have read their data. Tiles are handed out in increasing order by an atomic counter to a
// persistent grid, so every tile a warp waits for is already running on some other warp. The wait
// is bounded; on expiry the warp stores a code in *status and the kernel ends (its output is undefined).
//
// Scratch per row (zeroed before the launch), levels l = 0 .. L-1 with count[0] = tiles and
// count[l+1] = ceil(count[l] / 32): value (double) and flag (u32) per node, a counter (u32) per group.
#pragma once
#include "scan_kernels.cuh"

#define THB_SO_TILE 2048          // elements per warp tile: 16 float4 per lane
#define THB_SO_VECS 16
#define THB_SO_MAX_LEVELS 5       // 32^5 tiles of 2048 elements is far beyond any tensor
#define THB_SO_WAIT_NS 2000000000ull

struct ThbScanOnePass {
  const float* src;
  float* dst;
  long long n;              // row length (a multiple of 4)
  int rows;
  int levels;
  unsigned int count[THB_SO_MAX_LEVELS];     // nodes per level of one row
  unsigned int offset[THB_SO_MAX_LEVELS];    // first node of the level within a row's node arrays
  unsigned int nodes_per_row;                // sum of count[]
  double* value;            // [rows][nodes_per_row]
  unsigned int* flag;       // [rows][nodes_per_row]
  unsigned int* counter;    // [rows][nodes_per_row] (one per group of the level below; indexed like the parent node)
  unsigned int* next_tile;  // work counter
  int* status;
};

template <class Op>
__device__ __forceinline__ double thb_so_warp_fold(double v) {
  // lane order: ((l0 . l1) . (l2 . l3)) ... a fixed tree
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const double o = __shfl_down_sync(0xffffffffu, v, off);
    if (((threadIdx.x & 31) & (2 * off - 1)) == 0) v = Op::apply(v, o);
  }
  return __shfl_sync(0xffffffffu, v, 0);
}

template <class Op>
__global__ void __launch_bounds__(THB_SC_THREADS, 2)
thb_scan_rows_onepass(ThbScanOnePass P) {
  const int lane = threadIdx.x & 31;
  const unsigned int tiles_per_row = P.count[0];
  const unsigned long long total_tiles = (unsigned long long)tiles_per_row * P.rows;
  for (;;) {
    unsigned int tile = 0;
    if (lane == 0) tile = atomicAdd(P.next_tile, 1u);
    tile = __shfl_sync(0xffffffffu, tile, 0);
    if (tile >= total_tiles) return;
    const unsigned int row = tile / tiles_per_row, t = tile - row * tiles_per_row;
    const float* s = P.src + (long long)row * P.n + (long long)t * THB_SO_TILE;
    float* d = P.dst + (long long)row * P.n + (long long)t * THB_SO_TILE;
    const long long left = P.n - (long long)t * THB_SO_TILE;   // elements of the row from this tile on
    double* val = P.value + (size_t)row * P.nodes_per_row;
    unsigned int* flg = P.flag + (size_t)row * P.nodes_per_row;
    unsigned int* cnt = P.counter + (size_t)row * P.nodes_per_row;

    // ---- the tile: 16 float4 per lane, vector u of lane l = elements (u * 32 + l) * 4 .. + 3
    float4 v[THB_SO_VECS];
    const float idf = (float)Op::identity();
#pragma unroll
    for (int u = 0; u < THB_SO_VECS; ++u) {
      const int e = (u * 32 + lane) * 4;
      v[u] = e < left ? *reinterpret_cast<const float4*>(s + e) : make_float4(idf, idf, idf, idf);
    }
    // aggregate in the order of the elements: per vector, then lanes, then vectors
    double agg = Op::identity();
#pragma unroll
    for (int u = 0; u < THB_SO_VECS; ++u) {
      double x = Op::apply(Op::apply((double)v[u].x, (double)v[u].y), Op::apply((double)v[u].z, (double)v[u].w));
      agg = Op::apply(agg, thb_so_warp_fold<Op>(x));
    }

    // ---- publish, and complete groups upwards while this warp is the last of its group to arrive
    {
      unsigned int idx = t;
      double mine = agg;
      for (int l = 0; l < P.levels; ++l) {
        if (lane == 0) {
          val[P.offset[l] + idx] = mine;
          __threadfence();
          *((volatile unsigned int*)&flg[P.offset[l] + idx]) = 1u;
        }
        if (l + 1 >= P.levels) break;
        const unsigned int group = idx >> 5;
        const unsigned int members = min(32u, P.count[l] - (group << 5));
        unsigned int arrived = 0;
        if (lane == 0) {
          __threadfence();
          arrived = atomicAdd(&cnt[P.offset[l + 1] + group], 1u);
        }
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived != members - 1) break;          // somebody else will complete this group
        __threadfence();
        // every member's value is published: add them in lane order
        const double x = (unsigned int)lane < members ? __ldcg(&val[P.offset[l] + (group << 5) + lane]) : Op::identity();
        mine = thb_so_warp_fold<Op>(x);
        idx = group;
      }
    }

    // ---- carry-in: earlier nodes of this tile's group at every level, top level first
    double carry = Op::identity();
    bool ok = true;
    {
      unsigned int idx_at[THB_SO_MAX_LEVELS];
      idx_at[0] = t;
      for (int l = 1; l < P.levels; ++l) idx_at[l] = idx_at[l - 1] >> 5;
      for (int l = P.levels - 1; l >= 0 && ok; --l) {
        const unsigned int idx = idx_at[l];
        const unsigned int first = l + 1 < P.levels ? (idx >> 5) << 5 : 0u;   // the top level is one group
        const unsigned int need = idx - first;                                // earlier members of the group
        // (the top level has at most 32 nodes by construction)
        double x = Op::identity();
        if ((unsigned int)lane < need) {
          volatile unsigned int* f = (volatile unsigned int*)&flg[P.offset[l] + first + lane];
          if (*f == 0u) {
            unsigned long long t0;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
            for (unsigned int spin = 1; *f == 0u; ++spin) {
              if ((spin & 63u) == 0) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                if (now - t0 > THB_SO_WAIT_NS) { ok = false; break; }
              }
            }
          }
          if (ok) {
            __threadfence();
            x = __ldcg(&val[P.offset[l] + first + lane]);
          }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) carry = Op::apply(carry, thb_so_warp_fold<Op>(x));
      }
    }
    if (!ok) {
      if (lane == 0 && P.status) atomicCAS(P.status, 0, 3);
      return;
    }

    // ---- scan the tile from registers with the carry-in
    double run = carry;
#pragma unroll
    for (int u = 0; u < THB_SO_VECS; ++u) {
      const int e = (u * 32 + lane) * 4;
      double pre[4];
      pre[0] = (double)v[u].x;
      pre[1] = Op::apply(pre[0], (double)v[u].y);
      pre[2] = Op::apply(pre[1], (double)v[u].z);
      pre[3] = Op::apply(pre[2], (double)v[u].w);
      double incl = pre[3];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const double o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl = Op::apply(o, incl);
      }
      double excl = __shfl_up_sync(0xffffffffu, incl, 1);
      if (lane == 0) excl = Op::identity();
      const double before = Op::apply(run, excl);
      if (e < left)
        *reinterpret_cast<float4*>(d + e) = make_float4((float)Op::apply(before, pre[0]), (float)Op::apply(before, pre[1]),
                                                        (float)Op::apply(before, pre[2]), (float)Op::apply(before, pre[3]));
      run = Op::apply(run, __shfl_sync(0xffffffffu, incl, 31));
    }
  }
}
