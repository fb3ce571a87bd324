// Shared definitions of the stage-1 / stage-2 kernels: tile geometry, the split plan
// (evaluated identically on host and device) and small PTX helpers.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/fta.h"

#define FTA_TILE 64          // KV rows per tile, both kernel families
#define FTA_MAX_BATCH 8192   // prefix table lives in shared memory
#define FTA_LOG2E 1.4426950408889634f
#define FTA_LN2 0.6931471805599453f

// Geometry of one launch, computed on the host (fta_api.cu: make_geom).
// A "unit" is one (sequence b, KV head, M tile): the rows of M = G*Q query rows that one
// thread block multiplies against a stream of KV tiles.  An M tile is rectangular:
// hpt heads x qpt queries, row r -> (head r / qpt, query r % qpt).
struct FtaGeom {
  int R;       // rows of the kernel's M tile (16/32/64 mma, 128 umma)
  int qpt;     // queries per M tile
  int hpt;     // heads per M tile
  int n_qt;    // M tiles along Q
  int n_gt;    // M tiles along the group's heads
  int mtiles;  // n_qt * n_gt
  int U;       // units per sequence = Hkv * mtiles
  int n_tree;  // tree tiles per unit (0 when the tree is excluded)
  int grid;    // thread blocks launched (BALANCED: resident blocks)
  int min_per; // smallest tile range a block is given (BALANCED)
  int fixed_max_splits; // FIXED: ceil(ctx / split_tokens)
  int family;  // FTA_KERNEL_MMA or FTA_KERNEL_UMMA
  int cs;      // tcgen05 family: column split (2 when a unit has at most 64 query rows, else 1)
  int pad;     // BALANCED: what ending a unit costs a block, in tiles (see FtaBalanced)
  int lanes;   // BALANCED: blocks that walk the same tiles side by side, one M tile each (see FtaBalanced)
};

// One contiguous piece of one unit, processed by one block without interruption.
struct FtaSeg {
  int b;        // sequence
  int j;        // unit within the sequence: kvh * mtiles + mtile
  int c0, c1;   // cache rows [c0, c1)
  int tt0, tt1; // tree tiles [tt0, tt1)
  int split;    // index of this piece among the unit's pieces
  int nsplit;   // pieces of the unit (1 -> the block writes the final result itself)
  int slot;     // BALANCED: workspace slot of the partial
  int p0slot;   // BALANCED: workspace slot of the unit's first piece
};

__host__ __device__ __forceinline__ int fta_cdiv(int a, int b) { return (a + b - 1) / b; }

// kv_seq_len[b], clamped to [0, ctx].
__host__ __device__ __forceinline__ int fta_load_len(const void* lens, int is_i64, int b, int ctx) {
  long long v = is_i64 ? ((const long long*)lens)[b] : (long long)((const int*)lens)[b];
  if (v < 0) v = 0;
  if (v > ctx) v = ctx;
  return (int)v;
}

// ---- BALANCED plan ---------------------------------------------------------------------
// All units' tiles are laid on one line, sequence-major then unit then tile; a unit of
// sequence b has ceil(L_b/64) cache tiles, then n_tree tree tiles, then `pad` virtual tiles that
// stand for the work of ending a unit (last partial tile, tree tile, epilogue, pipeline restart):
// ut_b = real_b + pad, or 0 for a unit without real tiles.  pre[b] = sum_{b'<b} ut_b'.  Unit (b, j)
// starts at U*pre[b] + j*ut_b.  Block c owns the line positions [c*per, (c+1)*per), so blocks that
// end more units get fewer real tiles.  A unit whose real tiles are cut by k block boundaries has
// k+1 pieces; a range that covers only virtual tiles of a unit gives an empty piece, which callers skip.
//
// Lanes.  When a KV head's query rows need several M tiles (G*Q > rows of a tile), those units read
// the same K/V rows.  They are then not laid one after the other: the line holds one entry per KV
// head, `lanes` = M tiles per KV head, and blocks come in groups of `lanes` that own the same line
// range, block c working for M tile c % lanes.  The blocks of a group start together and walk the
// same tiles at the same pace, so all but the first request of a tile are served by L2 instead of
// DRAM.  Slots, pieces and cut descriptors stay per block; the pieces of one unit now sit `lanes`
// blocks apart.
__host__ __device__ __forceinline__ int fta_unit_tiles(int L, int n_tree, int pad) {
  const int real = (L + FTA_TILE - 1) / FTA_TILE + n_tree;
  return real > 0 ? real + pad : 0;
}
__host__ __device__ __forceinline__ bool fta_seg_empty(const FtaSeg& s) { return s.c1 <= s.c0 && s.tt1 <= s.tt0; }

struct FtaBalanced {
  const int* pre;  // [B+1]
  int B, U, n_tree, per, pad, lanes;  // U: entries per sequence on the line
  long long total;

  __host__ __device__ void init(const int* pre_, int B_, const FtaGeom& g, int grid) {
    pre = pre_; B = B_; n_tree = g.n_tree; pad = g.pad;
    lanes = g.lanes > 0 ? g.lanes : 1;
    U = g.U / lanes;
    total = (long long)U * pre[B];
    per = choose_per(total, grid / lanes > 0 ? grid / lanes : 1, g.min_per);
  }
  // line range [lin, end) of block c of `grid`; false if it has none
  __host__ __device__ bool range(int c, int grid, long long& lin, long long& end) const {
    if (c >= (grid / lanes) * lanes) return false;  // blocks left over after the last whole group
    lin = (long long)(c / lanes) * per;
    end = lin + per < total ? lin + per : total;
    return lin < end;
  }

  __host__ __device__ static int choose_per(long long total, int grid, int min_per) {
    long long per = (total + grid - 1) / (grid > 0 ? grid : 1);
    if (per < min_per) per = min_per;
    if (per < 1) per = 1;
    return (int)per;
  }

  // sequence whose tile range contains line position x (x < total)
  __host__ __device__ int find_b(long long x) const {
    int lo = 0, hi = B;  // invariant: U*pre[lo] <= x < U*pre[hi]
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if ((long long)U * pre[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
  }

  // Piece of block c that starts at line position lin (lin in c's range).  Returns the
  // line position where the piece ends.  I is the integer type of line positions: 32-bit
  // arithmetic when the whole line fits (64-bit division is slow on the device).
  template <typename I>
  __host__ __device__ long long segment_at_t(int cphys, I lin, FtaSeg& s) const {
    const int c = cphys / lanes, lane = cphys - c * lanes;  // group of blocks, M tile within the KV head
    const I cbeg = (I)c * (I)per;
    I cend = cbeg + (I)per;
    if (cend > (I)total) cend = (I)total;
    const int b = find_b((long long)lin);
    const int ut = pre[b + 1] - pre[b];
    const I boff = lin - (I)U * (I)pre[b];
    const int j = (int)(boff / (I)ut);
    const int t0 = (int)(boff - (I)j * (I)ut);
    const I ustart = lin - (I)t0, uend = ustart + (I)ut;
    const I send = cend < uend ? cend : uend;
    const int nreal = ut - pad;      // cache + tree tiles of this unit
    const int nb = nreal - n_tree;   // cache tiles
    int t1 = t0 + (int)(send - lin);
    const int r0 = t0 < nreal ? t0 : nreal;  // the real part of [t0, t1)
    t1 = t1 < nreal ? t1 : nreal;
    const int cfirst = (int)(ustart / (I)per), clast = (int)((ustart + (I)(nreal - 1)) / (I)per);
    s.b = b;
    s.j = j * lanes + lane;
    s.c0 = (r0 < nb ? r0 : nb) * FTA_TILE;
    s.c1 = (t1 < nb ? t1 : nb) * FTA_TILE;  // caller clamps to L_b
    s.tt0 = (r0 > nb ? r0 : nb) - nb;
    s.tt1 = (t1 > nb ? t1 : nb) - nb;
    if (s.tt1 < s.tt0) s.tt1 = s.tt0;
    s.split = c - cfirst;
    s.nsplit = clast - cfirst + 1;
    // A block holds at most two pieces of cut units: the one that opens its range (a later piece of
    // its unit: slot 0) and the one that closes it (the first piece of its unit: slot 1).  So every
    // piece's slot follows from the block that holds the unit's second piece, and stage 2 can ask for
    // the first two pieces before it has read the descriptor of the cut.
    s.slot = 2 * cphys + (c == cfirst ? 1 : 0);
    s.p0slot = 2 * (cfirst * lanes + lane) + 1;
    return (long long)send;
  }
  __host__ __device__ long long segment_at(int c, long long lin, FtaSeg& s) const {
    // positions up to total + per appear in the arithmetic
    if (total + per < 0x7fffffffLL) return segment_at_t<unsigned int>(c, (unsigned int)lin, s);
    return segment_at_t<long long>(c, lin, s);
  }
};

// ---- FIXED plan ------------------------------------------------------------------------
// Items are (b, j, s), s in [0, fixed_max_splits]; s < ceil(L_b/split_tokens) is a cache split,
// s == fixed_max_splits is the tree piece.  Items are dealt round-robin to the blocks (the walk
// is in each stage-1 kernel).

// ---- cache addressing --------------------------------------------------------------------
// Where cache rows [row0, row0 + 64) of sequence b start: for the dense cache (batch index b, row
// row0), for a paged one (page from the block table, row within the page).  row0 is a multiple of
// 64 and so is page_size, so a tile never straddles pages.
struct FtaTileAt {
  int batch;  // index along the cache's leading dimension
  int row;    // first row within it
};
__device__ __forceinline__ FtaTileAt fta_tile_at(const FtaParams& p, int b, int row0) {
  FtaTileAt t;
  if (p.block_table == nullptr) {
    t.batch = b; t.row = row0;
  } else {
    const int slot = row0 / p.page_size;
    t.batch = __ldg(p.block_table + (long long)b * p.bt_sb + slot);
    t.row = row0 - slot * p.page_size;
  }
  return t;
}

// ---- row <-> (head, query) mapping of an M tile -----------------------------------------
struct FtaUnit {
  int kvh, gt, qt;  // KV head, group-tile, query-tile
};
__host__ __device__ __forceinline__ FtaUnit fta_unit(const FtaGeom& g, int j) {
  FtaUnit u;
  u.kvh = j / g.mtiles;
  const int mt = j - u.kvh * g.mtiles;
  u.gt = mt / g.n_qt;
  u.qt = mt - u.gt * g.n_qt;
  return u;
}
// row r of the unit's tile -> head h and query qi; false if the row is padding
__host__ __device__ __forceinline__ bool fta_row(const FtaParams& p, const FtaGeom& g,
                                                 const FtaUnit& u, int r, int& h, int& qi) {
  const int hh = r / g.qpt;
  const int qq = r - hh * g.qpt;
  const int gi = u.gt * g.hpt + hh;
  qi = u.qt * g.qpt + qq;
  h = u.kvh * (p.H / p.Hkv) + gi;
  return hh < g.hpt && gi < (p.H / p.Hkv) && qi < p.Q;
}

#ifdef __CUDACC__
// ---- device helpers ----------------------------------------------------------------------

// BALANCED workspace: partial O rows [2*grid][R][D] fp32, partial LSEs [2*grid][R] fp32, then one
// int4 per stage-1 block: the unit whose SECOND piece opens that block, {b, j, pieces, slot of the
// first piece}, or pieces = 0.  Piece i >= 1 sits in slot 2*(block of the second piece + (i - 1)*lanes),
// piece 0 in slot 2*(block of the second piece - lanes) + 1.
// Stage 2 launches one group of blocks per stage-1 block and merges exactly the units that were cut.
__device__ __forceinline__ int4* fta_cut_desc(const FtaParams& p, const FtaGeom& g) {
  float* ws_o = reinterpret_cast<float*>(p.workspace);
  float* ws_l = ws_o + (long long)2 * g.grid * g.R * p.D;
  return reinterpret_cast<int4*>(ws_l + (long long)2 * g.grid * g.R);
}

// Block-cooperative build of the prefix table pre[0..B] in shared memory (warp 0 scans).
// Must be followed by __syncthreads().
__device__ __forceinline__ void fta_build_prefix(const FtaParams& p, int n_tree, int pad, int* pre) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int carry = 0;
    if (lane == 0) pre[0] = 0;
    for (int base = 0; base < p.B; base += 32) {
      const int b = base + lane;
      int v = 0;
      if (b < p.B) v = fta_unit_tiles(fta_load_len(p.kv_seq_len, p.len_is_i64, b, p.ctx), n_tree, pad);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
      }
      if (b < p.B) pre[b + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
}

__device__ __forceinline__ float fta_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fta_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> struct FtaType;
template <> struct FtaType<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ __half from_float(float a) { return __float2half_rn(a); }
};
template <> struct FtaType<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float a) { return __float2bfloat16_rn(a); }
};

// Store 4 consecutive output values (fp32 in registers) as `out_dtype` at element
// offset `off` of `base`.  off is a multiple of 4.
__device__ __forceinline__ void fta_store4(void* base, int out_dtype, long long off, float4 v) {
  if (out_dtype == FTA_DTYPE_F32) {
    *reinterpret_cast<float4*>((float*)base + off) = v;
  } else if (out_dtype == FTA_DTYPE_F16) {
    uint2 w;
    w.x = FtaType<__half>::pack(v.x, v.y);
    w.y = FtaType<__half>::pack(v.z, v.w);
    *reinterpret_cast<uint2*>((__half*)base + off) = w;
  } else {
    uint2 w;
    w.x = FtaType<__nv_bfloat16>::pack(v.x, v.y);
    w.y = FtaType<__nv_bfloat16>::pack(v.z, v.w);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)base + off) = w;
  }
}
#endif  // __CUDACC__
