// Stage 1, tcgen05 family: split-KV tree attention with both products on the 5th-generation
// tensor cores.  One thread block owns one M tile of 128 rows (all tree queries x the GQA
// heads that share a KV head) and streams 64-row KV tiles.  384 threads, three warpgroups:
//
//   warp 0      TMA producer: Q once per piece of work (two 4-D copies), then one 5-D copy per K
//               and per V tile (64 rows x 2 halves of 64 columns, 128-byte swizzle) into a 5- or
//               6-stage ring guarded by mbarriers; K tiles are requested two tiles ahead of V tiles
//   warp 1      issuer of S = Q K^T (128x64, fp32 in TMEM, three buffers, up to three tiles ahead
//               of the softmax)
//   warp 2      issuer of O += P V (128x128, fp32 in TMEM).  The A operands Q and P are read
//               from TMEM, so only K and V cross shared memory; completion of either product is
//               signalled by tcgen05.commit.  Two issuers because one thread cannot feed the
//               tensor pipe with 12 small products per tile and answer five barriers in time
//   warp 3      planner: walks the block's pieces of work once and hands each to the other roles
//               as a 64-byte descriptor in a shared-memory ring
//   warps 4..7  softmax: a thread owns one row (TMEM lane); per tile tcgen05.ld of S, scale, tree
//               mask / sequence-end mask, running max with lazy rescale of O, exp2 (a quarter of them on
//               the FMA pipe), P (16-bit pairs) stored to TMEM over the S columns just read; at the
//               end of a piece the row's maximum and sum go to the epilogue warps through two TMEM
//               columns and the next piece starts (with two Q buffers its first S tiles are waiting)
//   warps 8..11 epilogue: a thread owns one row; where TMEM has room for two Q buffers (no tile
//               pairs, no column split) it copies the Q row of the NEXT piece from shared memory into
//               the other buffer while the current piece is worked on (else the softmax thread copies
//               it at the start of the piece); reads a finished piece's O rows from TMEM (handing the
//               accumulator back at once), normalises, stages through the Q buffer and stores 256-byte
//               row pieces, and the LSE; all of it beside the next piece's tiles
//
// Registers are rebalanced with setmaxnreg (64 per thread for warps 0..3, 240 for the softmax, 200
// for the epilogue).
//
// Tile pairs (template PAIRS, no column split): the softmax takes full cache tiles two at a time, so
// that everything that costs a round trip is paid once per 128 KV rows; four S buffers, P written
// over the S columns just read.  Chosen by the launcher where blocks are fed through L2.
//
// Column split (template CS = 2): when a unit has at most 64 query rows (q_len 64 without GQA),
// rows 64..127 of the tile repeat rows 0..63 (Q is loaded twice) and each half of the tile's rows
// works on its own 32 of every tile's 64 KV columns, with its own running max, row sum and O rows.
// Half of each P row is then zero, the two O halves are two partial attentions of the same query
// and are merged through shared memory by the epilogue warps.  The tensor work is unchanged (the
// tile has 128 rows either way) but all four schedulers share the exponentials.
//
// It replaces the reference's _flash_decoding_fwd_kernel (flash_tree_attn.py:14-144) and the
// eager tree tail (flash_tree_attn.py:367-371) for head_dim 128 when M = G*Q is large enough
// to fill a 128-row tile usefully; the work plan and the partial-result slots are those of the
// warp-MMA family.
//
// Every mbarrier wait is bounded (fta_umma_ptx.cuh); on a timeout the block records a code in
// g_umma_status, all roles leave their loops, and the block still frees its TMEM.
#include <mutex>

#include "fta_common.cuh"
#include "fta_umma_ptx.cuh"

namespace fta_umma {

constexpr int kThreads = 384;  // warps 0-3: TMA producer, QK issuer, PV issuer, planner; 4-7 softmax; 8-11 epilogue
// Registers per thread after the warpgroups have rebalanced (the block is launched with 168 each)
constexpr int kRegsIssue = 64, kRegsSoftmax = 240, kRegsEpilogue = 200;
constexpr int kD = 128;
constexpr int kR = 128;
constexpr uint32_t kQHalf = kR * 128;         // 128 rows x 64 elements
constexpr uint32_t kQBytes = 2 * kQHalf;
constexpr uint32_t kKVHalf = FTA_TILE * 128;  // 64 rows x 64 elements
constexpr uint32_t kKBytes = 2 * kKVHalf;
constexpr uint32_t kStage = 2 * kKBytes;      // K tile then V tile
constexpr uint32_t OFF_Q = 0;
constexpr uint32_t OFF_RING = OFF_Q + kQBytes;
constexpr uint32_t kBarBytes = 512;
constexpr int kSegRing = 8;                  // pieces of work the planner may run ahead
constexpr uint32_t kSegBytes = kSegRing * 64;
// TMEM columns (32-bit).  Several S buffers let S = Q K^T run ahead of the softmax.  A thread has
// all of its S row in registers before it writes P, so P(t) (16-bit pairs) goes over the first 32
// columns of S(t); S(t) is not issued before PV(t - buffers), which read that P, is complete.
//   three buffers:  O fp32 0..127 | S/P 128 + 64 k (k < 3) | Q of even pieces 320..383 | Q of odd
//                   pieces 384..447 | row statistics 480..481.  With two Q buffers the next piece's Q
//                   rows are in TMEM long before the piece starts, so its first products are issued
//                   behind the last ones of the piece before and S never runs dry at a boundary.
//   three buffers, column split (CS = 2):  O 0..127 | S 128 + 64 k | Q 320..383 (one buffer) | P
//                   384 + 32 k, apart from S: the half of a P row that belongs to the other half of
//                   the tile's rows is zeroed once and never written again | statistics 480..481.
//   four buffers (template PAIRS, where the softmax takes full tiles two at a time):  O 0..127 |
//                   S/P 128 + 64 k (k < 4) | Q 384..447 (one buffer: no room for two) | row
//                   statistics 448..449.
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxBuf = 4;
__host__ __device__ constexpr int n_buf(bool pairs) { return pairs ? 4 : 3; }
constexpr uint32_t kColS = 128;  // + 64 * buffer
__host__ __device__ constexpr int n_qbuf(bool pairs, int cs) { return (pairs || cs == 2) ? 1 : 2; }
// 64 columns per buffer: 128 head-dim elements, two per column
__host__ __device__ constexpr uint32_t col_q(bool pairs, int cs, uint32_t piece) {
  return pairs ? 384u : 320u + (cs == 2 ? 0u : 64u * (piece & 1u));
}
__host__ __device__ constexpr uint32_t col_p(bool, int cs, uint32_t buf) { return cs == 2 ? 384u + 32u * buf : kColS + 64u * buf; }
__host__ __device__ constexpr uint32_t col_stat(bool pairs) { return pairs ? 448u : 480u; }
// shared-memory size of a block with NS ring stages and a B-entry prefix table
constexpr uint32_t kXBytes = 2 * 64 * 64 * 4 + 2 * 64 * 2 * 4;  // CS = 2: per half 64 rows x 64 unnormalised O columns, and (m, l) per row
constexpr size_t smem_bytes(int ns, int B, int cs) {
  return (size_t)OFF_RING + (size_t)ns * kStage + (cs == 2 ? kXBytes : 0) + kBarBytes + kSegBytes + (size_t)(B + 1) * 4 + (cs == 2 ? 0 : 1024);
}

// mbarrier slots (ring barriers are sized for the largest ring)
constexpr int kMaxNS = 6;
enum { B_QFULL = 0, B_QEMPTY, B_QREADY, B_ODONE = B_QREADY + 2, B_OFREE = B_ODONE + 4, B_KFULL, B_VFULL = B_KFULL + kMaxNS,
       B_KEMPTY = B_VFULL + kMaxNS, B_VEMPTY = B_KEMPTY + kMaxNS, B_SFULL = B_VEMPTY + kMaxNS, B_PREADY = B_SFULL + kMaxBuf,
       B_FINAL = B_PREADY + kMaxBuf, B_XFULL = B_FINAL + 2, B_XFREE, B_SEGFULL, B_SEGFREE = B_SEGFULL + kSegRing,
       B_STATS = B_SEGFREE + kSegRing, B_STATSFREE, B_COUNT };
// A parity wait is only meaningful while the barrier is at most one phase ahead of the phase
// asked for.  PV(t) therefore commits to B_ODONE + (t & 3): whoever has seen S(t') ready knows
// that PV(t'-4) and everything before it is complete, so for t in [t'-3, t'] the barrier of PV(t)
// has completed phase (t>>2)-1 and cannot have completed more than phase t>>2.
static_assert(B_COUNT * 8 + 8 <= kBarBytes, "barrier area");

struct Maps {
  CUtensorMap q, k, v, ck, cv;
};

// Walks this block's pieces of work, identically in every role.
struct Walker {
  const FtaParams& p;
  const FtaGeom& g;
  FtaBalanced plan;
  long long lin, lin_end, item, n_items;
  __device__ Walker(const FtaParams& p_, const FtaGeom& g_, const int* pre) : p(p_), g(g_) {
    lin = lin_end = item = n_items = 0;
    if (p.split_mode == FTA_SPLIT_BALANCED) {
      plan.init(pre, p.B, g, gridDim.x);
      if (!plan.range(blockIdx.x, gridDim.x, lin, lin_end)) lin = lin_end = 0;
    } else {
      item = blockIdx.x;
      n_items = (long long)p.B * g.U * (g.fixed_max_splits + 1);
    }
  }
  __device__ bool next(FtaSeg& seg) {
    if (p.split_mode == FTA_SPLIT_BALANCED) {
      do {  // ranges that cover only the virtual tail of a unit hold no work
        if (lin >= lin_end) return false;
        lin = plan.segment_at(blockIdx.x, lin, seg);
      } while (fta_seg_empty(seg));
      const int Lb = fta_load_len(p.kv_seq_len, p.len_is_i64, seg.b, p.ctx);
      if (seg.c1 > Lb) seg.c1 = Lb;
      return true;
    }
    const int per_unit = g.fixed_max_splits + 1;
    const long long per_b = (long long)g.U * per_unit;
    while (item < n_items) {
      seg.b = (int)(item / per_b);
      const long long r = item - (long long)seg.b * per_b;
      seg.j = (int)(r / per_unit);
      seg.split = (int)(r - (long long)seg.j * per_unit);
      item += gridDim.x;
      seg.nsplit = 0; seg.slot = 0;
      const int Lb = fta_load_len(p.kv_seq_len, p.len_is_i64, seg.b, p.ctx);
      if (seg.split == g.fixed_max_splits) {
        if (g.n_tree == 0) continue;
        seg.c0 = seg.c1 = 0; seg.tt0 = 0; seg.tt1 = g.n_tree;
        return true;
      }
      seg.c0 = seg.split * p.split_tokens;
      if (seg.c0 >= Lb) continue;
      seg.c1 = seg.c0 + p.split_tokens < Lb ? seg.c0 + p.split_tokens : Lb;
      seg.tt0 = seg.tt1 = 0;
      return true;
    }
    return false;
  }
};

// One piece of work as the planner warp hands it to the other roles (shared memory, 64 bytes).
struct __align__(16) SegDesc {
  int valid;            // 0: the block has no more work
  int b, kvh, gt, qt;   // sequence; KV head, group tile and query tile of the unit
  int c0, c1;           // cache rows [c0, c1), c1 already clamped to the sequence length
  int tt0, tt1;         // tree tiles [tt0, tt1)
  int split, nsplit, slot, p0slot, j;
  int pad[2];
};
static_assert(sizeof(SegDesc) == 64, "descriptor size");

// Warp-collective wait: every lane gets the same answer, so the lanes of a warp leave their loops
// together (the TMEM loads that follow are warp-wide instructions).
__device__ __forceinline__ bool wait_all(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, code)) != 0;
}

__device__ __forceinline__ int seg_cache_tiles(const SegDesc& s) {
  return s.c1 > s.c0 ? fta_cdiv(s.c1 - s.c0, FTA_TILE) : 0;
}
__device__ __forceinline__ void seg_copy(SegDesc& d, const SegDesc* src) {
  const int4* s4 = reinterpret_cast<const int4*>(src);
  int4* d4 = reinterpret_cast<int4*>(&d);
#pragma unroll
  for (int i = 0; i < 4; ++i) d4[i] = s4[i];
}

template <typename T, int NS, int CS, bool PAIRS>
__global__ void __launch_bounds__(kThreads, 1)
stage1_umma_kernel(const FtaParams p, const FtaGeom g, const __grid_constant__ Maps maps) {
  constexpr uint32_t OFF_X = OFF_RING + NS * kStage;
  constexpr uint32_t OFF_BAR = OFF_X + (CS == 2 ? kXBytes : 0);
  constexpr uint32_t OFF_SEG = OFF_BAR + kBarBytes;
  static_assert(!(PAIRS && CS == 2), "tiles are taken in pairs only without the column split");
  constexpr int kNBuf = n_buf(PAIRS);
  constexpr uint32_t kColStat = col_stat(PAIRS);
  constexpr int kQBuf = n_qbuf(PAIRS, CS);
  constexpr uint32_t OFF_PRE = OFF_SEG + kSegBytes;
  // Swizzle atoms are 1024-byte aligned.  Without the column split there is room to round the base
  // up; with it every kilobyte is taken, the declared alignment is relied on and checked.
  extern __shared__ uint8_t smem_plain[];
  extern __shared__ __align__(1024) uint8_t smem_aligned[];  // the same memory, alignment declared
  uint8_t* smem_raw;
  if constexpr (CS == 2) smem_raw = smem_aligned; else smem_raw = smem_plain;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = CS == 2 ? raw : ((raw + 1023u) & ~1023u);
  if (CS == 2 && (base & 1023u)) {  // never seen; without the alignment nothing below may run
    if (threadIdx.x == 0) atomicCAS(&g_umma_status, 0u, 0x7ffu);
    return;
  }
  uint8_t* sm = smem_raw + (base - raw);
  int* pre = reinterpret_cast<int*>(sm + OFF_PRE);
  SegDesc* segq = reinterpret_cast<SegDesc*>(sm + OFF_SEG);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_BAR + kBarBytes - 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_BAR + kBarBytes - 4);
  const uint32_t bar0 = base + OFF_BAR;
#define BAR(i) (bar0 + 8u * (uint32_t)(i))
  // Q(piece) is announced on one barrier per TMEM buffer, so that a waiter can never be two phases behind
  auto qready_bar = [&](uint32_t piece) -> uint32_t { return BAR(B_QREADY + (kQBuf == 2 ? (piece & 1u) : 0u)); };
  auto qready_par = [&](uint32_t piece) -> uint32_t { return (kQBuf == 2 ? (piece >> 1) : piece) & 1u; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef FTA_UMMA_PROFILE
  const long long prof_t0 = clock64();
  if (blockIdx.x == 0 && threadIdx.x == 0) g_umma_trace_t0 = prof_t0;
  unsigned long long prof_g0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_g0));
#endif
  const int G = p.H / p.Hkv;
  const int fmt = p.dtype == FTA_DTYPE_BF16 ? 1 : 0;

  // stage 2 is launched with programmatic stream serialization: let its grid be set up now; its
  // blocks wait for this whole grid to finish before they read anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the copy engine's descriptors are fetched while the block sets itself up
  if (tid == 32 * 0 + 31) {
    tma_prefetch_desc(&maps.q); tma_prefetch_desc(&maps.k); tma_prefetch_desc(&maps.v);
    if (g.n_tree) { tma_prefetch_desc(&maps.ck); tma_prefetch_desc(&maps.cv); }
  }

  // one barrier per thread: slot i expects count(i) arrivals per phase
  if (tid < B_COUNT) {
    uint32_t count = 1;
    if (tid == B_QEMPTY || tid == B_QREADY || tid == B_QREADY + 1 || tid == B_OFREE || tid == B_STATS || tid == B_STATSFREE ||
        (tid >= B_PREADY && tid < B_PREADY + kNBuf))
      count = 128;
    else if (tid == B_XFULL || tid == B_XFREE) count = 128;
    else if (tid >= B_SEGFREE && tid < B_SEGFREE + kSegRing) count = 4;
    mbar_init(BAR(tid), count);
    fence_barrier_init();
  }
  if (tid == 0) *abort_flag = 0;
  // Q rows the TMA box never covers (M tile padding) must read as zero; the epilogue, which
  // borrows the buffer, leaves them alone too.
  {
    const uint32_t box_rows = (uint32_t)(g.qpt * g.hpt);
    for (uint32_t i = tid; i < kQBytes / 16; i += kThreads) {
      const uint32_t r = (i >> 3) & (kR - 1);  // [half][row][8 chunks]
      if ((r & (kR / CS - 1)) >= box_rows) reinterpret_cast<uint4*>(sm + OFF_Q)[i] = make_uint4(0, 0, 0, 0);
    }
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  // Everything above is local to the block.  If this grid was launched to overlap the kernel before it
  // in the stream, that kernel (and whatever it waited for) has finished once this returns; nothing in
  // global memory is read or written before.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (p.split_mode == FTA_SPLIT_BALANCED) fta_build_prefix(p, g.n_tree, g.pad, pre);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (tid == 0) FTA_TRACE_EP(12, 0);

  // Q row of a thread (row = its TMEM lane): shared memory (TMA, swizzled) -> TMEM, 16-bit pairs, one
  // per column.  One Q buffer: the softmax warps do it at the start of a piece, when every S = Q K^T of
  // the piece before is complete (its last S has been read).  Two Q buffers: the epilogue warps do it,
  // because they are idle while a piece's tiles are worked on, so the next piece's rows are in place
  // well before that piece's first product is due; the buffer they write was last read by the products
  // of the piece before the current one, which they have seen complete.
  auto q_to_tmem = [&](int row, uint32_t t_lane, uint32_t piece) -> bool {
    if (!wait_all(BAR(B_QFULL), piece & 1, abort_flag, 0x306)) return false;
    if (row == 0 && piece == 0) FTA_TRACE_EP(12, 4);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      uint32_t qr[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(sm + OFF_Q + hf * kQHalf + row * 128 + ((c ^ (row & 7)) << 4));
        qr[4 * c] = v.x; qr[4 * c + 1] = v.y; qr[4 * c + 2] = v.z; qr[4 * c + 3] = v.w;
      }
      tmem_st32(t_lane + col_q(PAIRS, CS, piece) + 32 * hf, reinterpret_cast<const float*>(qr));
    }
    tmem_st_wait();
    tc_fence_before();
    mbar_arrive(qready_bar(piece));
    if (row == 0 && piece == 0) FTA_TRACE_EP(12, 5);
    return true;
  };

  if (warp < 4) {
    reg_dec<kRegsIssue>();
    if (warp == 3) {
      // ================================ planner =====================================
      // Walks this block's pieces of work once, for everybody: the lookup (a search in the prefix
      // table, divisions, a sequence length from global memory) is off every other role's path.
      if (lane == 0) {
        Walker w(p, g, pre);
        FtaSeg seg;
        for (uint32_t k = 0;; ++k) {
          const bool have = w.next(seg);
          const uint32_t slot = k % kSegRing;
          if (k >= kSegRing && !mbar_wait(BAR(B_SEGFREE + slot), ((k / kSegRing) - 1) & 1, abort_flag, 0x402)) break;
          SegDesc d;
          d.valid = have ? 1 : 0;
          if (have) {
            const FtaUnit unit = fta_unit(g, seg.j);
            d.b = seg.b; d.kvh = unit.kvh; d.gt = unit.gt; d.qt = unit.qt;
            d.c0 = seg.c0; d.c1 = seg.c1; d.tt0 = seg.tt0; d.tt1 = seg.tt1;
            d.split = seg.split; d.nsplit = seg.nsplit; d.slot = seg.slot; d.p0slot = seg.p0slot; d.j = seg.j;
          } else {
            d.b = d.kvh = d.gt = d.qt = d.c0 = d.c1 = d.tt0 = d.tt1 = d.split = d.nsplit = d.slot = d.p0slot = d.j = 0;
          }
          d.pad[0] = d.pad[1] = 0;
          int4* dst = reinterpret_cast<int4*>(&segq[slot]);
          const int4* src = reinterpret_cast<const int4*>(&d);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = src[i];
          mbar_arrive(BAR(B_SEGFULL + slot));  // release: the descriptor is visible to whoever sees the phase
          if (k == 0) FTA_TRACE_EP(12, 1);
          if (!have) break;
        }
      }
    } else if (warp == 0) {
      // ================================ TMA producer ================================
      if (lane == 0) {
        uint32_t gt = 0;
        bool ok = true;
        for (uint32_t sidx = 0; ok; ++sidx) {
          SegDesc seg;
          ok = mbar_wait(BAR(B_SEGFULL + sidx % kSegRing), (sidx / kSegRing) & 1, abort_flag, 0x100);
          if (!ok) break;
          seg_copy(seg, &segq[sidx % kSegRing]);
          if (!seg.valid) break;
          const int n_ct = seg_cache_tiles(seg), n = n_ct + seg.tt1 - seg.tt0;
          const int q_at = sidx == 0 ? 0 : (n < 2 ? n : 2);  // nothing to overlap before the first piece: its Q goes first
          if (sidx == 0) FTA_TRACE_EP(12, 2);
          // K tiles run two ahead of V tiles, as their consumers (S = Q K^T, O += P V) do.  The
          // first K tiles of a piece are requested before its Q tile: they do not depend on the
          // Q buffer having been handed back, so they overlap the previous piece's tail.  (The
          // block's first piece has no predecessor and the first S waits for Q: there Q leads.)
          // Paged cache: a tile's page comes from the block table.  The entry for tile u + 1 is
          // requested while tile u is being issued, and a tile's entry is kept for its V copy two
          // iterations later, so that no copy waits for a table read.
          FtaTileAt at_m2 = {0, 0}, at_m1 = {0, 0}, at_0 = {0, 0}, at_p1 = {0, 0};  // tiles u - 2, u - 1, u, u + 1
          if (n_ct > 0) at_0 = fta_tile_at(p, seg.b, seg.c0);
          for (int u = 0; u < n + 2 && ok; ++u) {
            if (u > 0) { at_m2 = at_m1; at_m1 = at_0; at_0 = at_p1; }
            if (u + 1 < n_ct) at_p1 = fta_tile_at(p, seg.b, seg.c0 + (u + 1) * FTA_TILE);
            if (u == q_at) {
              ok = mbar_wait(BAR(B_QEMPTY), (sidx & 1) ^ 1, abort_flag, 0x101);
              if (!ok) break;
              mbar_expect_tx(BAR(B_QFULL), 2u * CS * (uint32_t)(g.qpt * g.hpt) * 128u);
              if (sidx == 0) FTA_TRACE_EP(12, 3);
              const int h0 = seg.kvh * G + seg.gt * g.hpt, q0 = seg.qt * g.qpt;
#pragma unroll
              for (int dup = 0; dup < CS; ++dup) {  // CS = 2: the same rows again at tile rows 64..
                tma_load_4d(base + OFF_Q + dup * 64 * 128, &maps.q, BAR(B_QFULL), 0, q0, h0, seg.b);
                tma_load_4d(base + OFF_Q + kQHalf + dup * 64 * 128, &maps.q, BAR(B_QFULL), 64, q0, h0, seg.b);
              }
            }
            for (int which = 0; which < 2; ++which) {  // 0: K of tile u, 1: V of tile u - 2
              const int i = which == 0 ? u : u - 2;
              if (i < 0 || i >= n) continue;
              const uint32_t t = gt + i, st = t % NS;
              const CUtensorMap* m;
              int row0, head, bidx = seg.b;
              if (i < n_ct) {
                const FtaTileAt at = which == 0 ? at_0 : at_m2;  // dense: (b, row); paged: (page, row in page)
                m = which == 0 ? &maps.k : &maps.v; row0 = at.row; bidx = at.batch; head = seg.kvh;
              } else { m = which == 0 ? &maps.ck : &maps.cv; row0 = (seg.tt0 + i - n_ct) * FTA_TILE; head = seg.kvh * p.cur_head_mul; }
              const uint32_t full = BAR((which == 0 ? B_KFULL : B_VFULL) + st);
              ok = mbar_wait(BAR((which == 0 ? B_KEMPTY : B_VEMPTY) + st), ((t / NS) & 1) ^ 1, abort_flag, 0x102 + which);
              if (!ok) break;
              const uint32_t dst = base + OFF_RING + st * kStage + (which == 0 ? 0u : kKBytes);
              FTA_TRACE(t, which);
              mbar_expect_tx(full, kKBytes);
              tma_load_5d(dst, m, full, 0, row0, head, 0, bidx);
            }
          }
          gt += n;
        }
      }
    } else if (warp == 1) {
      // ================================ S = Q K^T issuer ============================
      // The whole warp walks the loop (uniform control flow keeps descriptor arithmetic cheap);
      // one elected lane issues.  S(t) goes to buffer t%3 as soon as the softmax has finished
      // reading S(t-3), so the products run up to three tiles ahead of the softmax.
      const uint32_t idesc_qk = instr_desc_f16(fmt, kR, FTA_TILE, 0, 0);
      const uint64_t dK0 = smem_desc_sw128(base + OFF_RING, 16, 1024);
      uint32_t gt = 0;
      bool ok = true;
      for (uint32_t sidx = 0; ok; ++sidx) {
        SegDesc seg;
        ok = wait_all(BAR(B_SEGFULL + sidx % kSegRing), (sidx / kSegRing) & 1, abort_flag, 0x200);
        if (!ok) break;
        seg_copy(seg, &segq[sidx % kSegRing]);
        if (!seg.valid) break;
        const int n = seg_cache_tiles(seg) + seg.tt1 - seg.tt0;
        ok = wait_all(qready_bar(sidx), qready_par(sidx), abort_flag, 0x201);  // Q rows are in TMEM
        const uint32_t q_tmem = tmem + col_q(PAIRS, CS, sidx);
        if (lane == 0 && sidx == 0) FTA_TRACE_EP(12, 6);
        if (lane == 0 && sidx > 0) FTA_TRACE_EP(sidx - 1, 5);
        for (int i = 0; i < n && ok; ++i) {
          const uint32_t t = gt + i, st = t % NS, sbuf = t % kNBuf;
          if (t >= kNBuf) {
            // S[t%3] has been read by softmax(t-3); and PV(t-3) is complete, so that whoever sees
            // S(t) ready may overwrite P[t%3] without asking.  Both happened about two tiles ago.
            ok = wait_all(BAR(B_PREADY + sbuf), ((t - kNBuf) / kNBuf) & 1, abort_flag, 0x204);
            if (!ok) break;
            ok = wait_all(BAR(B_ODONE + ((t - kNBuf) & 3)), ((t - kNBuf) >> 2) & 1, abort_flag, 0x207);
            if (!ok) break;
          }
          ok = wait_all(BAR(B_KFULL + st), (t / NS) & 1, abort_flag, 0x202);
          if (!ok) break;
          if (lane == 0 && sidx > 0 && i == 0) FTA_TRACE_EP(sidx - 1, 7);
          tc_fence_after();
          if (elect_one()) {
            FTA_TRACE(t, 2);
            const uint64_t dK = dK0 + (uint64_t)((st * kStage) >> 4);
            const uint32_t d_tmem = tmem + kColS + FTA_TILE * sbuf;
#pragma unroll
            for (int ks = 0; ks < kD / 16; ++ks) {
              const uint32_t half = ks >> 2, off = (ks & 3) * 32;
              umma_f16_ts(d_tmem, q_tmem + ks * 8, dK + (uint64_t)((half * kKVHalf + off) >> 4), idesc_qk, ks > 0);
            }
            umma_commit(BAR(B_KEMPTY + st));
            umma_commit(BAR(B_SFULL + sbuf));
          }
          __syncwarp();
        }
        gt += n;
      }
      // nothing of this warp's may still be running on the tensor pipe when TMEM is freed
      if (elect_one()) umma_commit(BAR(B_FINAL));
      __syncwarp();
      int zero = 0;
      mbar_wait(BAR(B_FINAL), 0, &zero, 0x20f);
    } else {
      // ================================ O += P V issuer =============================
      const uint32_t idesc_pv = instr_desc_f16(fmt, kR, kD, 0, 1);
      const uint64_t dV0 = smem_desc_sw128(base + OFF_RING + kKBytes, kKVHalf, 1024);
      uint32_t gt = 0;
      bool ok = true;
      for (uint32_t sidx = 0; ok; ++sidx) {
        SegDesc seg;
        ok = wait_all(BAR(B_SEGFULL + sidx % kSegRing), (sidx / kSegRing) & 1, abort_flag, 0x210);
        if (!ok) break;
        seg_copy(seg, &segq[sidx % kSegRing]);
        if (!seg.valid) break;
        const int n = seg_cache_tiles(seg) + seg.tt1 - seg.tt0;
        for (int i = 0; i < n && ok; ++i) {
          const uint32_t t = gt + i, st = t % NS, sbuf = t % kNBuf;
          ok = wait_all(BAR(B_PREADY + sbuf), (t / kNBuf) & 1, abort_flag, 0x214);  // P(t) is in TMEM
          if (!ok) break;
          if (lane == 0) FTA_TRACE(t, 6);
          ok = wait_all(BAR(B_VFULL + st), (t / NS) & 1, abort_flag, 0x215);
          if (!ok) break;
          if (lane == 0) FTA_TRACE(t, 7);
          if (i == 0) {  // the previous piece's epilogue must have read O
            ok = wait_all(BAR(B_OFREE), (sidx & 1) ^ 1, abort_flag, 0x216);
            if (!ok) break;
          }
          tc_fence_after();
          if (elect_one()) {
            const uint64_t dV = dV0 + (uint64_t)((st * kStage) >> 4);
#pragma unroll
            for (int kk = 0; kk < FTA_TILE / 16; ++kk)
              umma_f16_ts(tmem, tmem + col_p(PAIRS, CS, sbuf) + kk * 8, dV + (uint64_t)((kk * 16 * 128) >> 4), idesc_pv,
                          (i > 0 || kk > 0) ? 1u : 0u);
            umma_commit(BAR(B_VEMPTY + st));
            umma_commit(BAR(B_ODONE + (t & 3)));
          }
          __syncwarp();
        }
        gt += n;
      }
      if (elect_one()) umma_commit(BAR(B_FINAL + 1));
      __syncwarp();
      int zero = 0;
      mbar_wait(BAR(B_FINAL + 1), 0, &zero, 0x21f);
    }
  } else if (warp < 8) {
    // ================================ softmax =======================================
    reg_inc<kRegsSoftmax>();
    const int quad = warp & 3;  // the TMEM lane quadrant a warp may touch is fixed by its index
    const int row = quad * 32 + lane;
    constexpr int NC = FTA_TILE / CS;            // KV columns of a tile this thread works on
    const int lrow = CS == 2 ? (row & 63) : row;  // query row of the unit this thread works for
    const int chalf = CS == 2 ? (row >> 6) : 0;  // which NC columns of each tile
    const int cbase = NC * chalf;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
    if (CS == 2) {
      // the half of every P row this thread never writes must read as zero
      uint32_t z[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) z[k] = 0u;
#pragma unroll
      for (int k = 0; k < kNBuf; ++k) tmem_st16(t_lane + col_p(PAIRS, CS, k) + 16 * (chalf ^ 1), z);
      tmem_st_wait();
      tc_fence_before();
    }
    const float scale2 = p.sm_scale * FTA_LOG2E;
    uint32_t gt = 0, sidx = 0;
    bool ok = true;

    // V rows past the end of the sequence are zeroed so that 0 * padding cannot give NaN
    auto zero_v_tail = [&](uint32_t t, int valid) -> bool {
      const uint32_t st = t % NS;
      if (!wait_all(BAR(B_VFULL + st), (t / NS) & 1, abort_flag, 0x303)) return false;
      uint8_t* sV = sm + OFF_RING + st * kStage + kKBytes;
      const int nz = (FTA_TILE - valid) * 16;
      for (int idx = row; idx < nz; idx += 128) {
        const int rr = valid + (idx >> 4), hc = idx & 15;
        *reinterpret_cast<uint4*>(sV + (hc >> 3) * kKVHalf + rr * 128 + (hc & 7) * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async();
      return true;
    };

    SegDesc seg;
    ok = wait_all(BAR(B_SEGFULL), 0, abort_flag, 0x300);
    if (ok) {
      seg_copy(seg, &segq[0]);
      if (kQBuf == 1 && seg.valid) ok = q_to_tmem(row, t_lane, 0);
    } else {
      seg.valid = 0;
    }
    while (ok && seg.valid) {
      FtaUnit unit;
      unit.kvh = seg.kvh; unit.gt = seg.gt; unit.qt = seg.qt;
      const int n_ct = seg_cache_tiles(seg), n = n_ct + seg.tt1 - seg.tt0;
      int h, qi;
      const bool rvalid = fta_row(p, g, unit, lrow, h, qi);
      const float* mrow = (rvalid && g.n_tree) ? p.mask + seg.b * p.m_sb + h * p.m_sh + qi * p.m_sq : nullptr;
      float m_used = -INFINITY, l = 0.f;
      const bool working = __any_sync(0xffffffffu, rvalid) != 0;

      if (!working) {
        // a warp whose 32 rows are all M-tile padding only keeps the barrier protocol going
        for (int i = 0; i < n; ++i) {
          const uint32_t t = gt + i, sbuf = t % kNBuf;
          ok = wait_all(BAR(B_SFULL + sbuf), (t / kNBuf) & 1, abort_flag, 0x311);
          if (!ok) break;
          if (i < n_ct) {
            const int row0 = seg.c0 + i * FTA_TILE;
            const int valid = seg.c1 - row0 < FTA_TILE ? seg.c1 - row0 : FTA_TILE;
            if (valid < FTA_TILE) {
              ok = zero_v_tail(t, valid);
              if (!ok) break;
            }
          }
          mbar_arrive(BAR(B_PREADY + sbuf));
        }
        if (!ok) break;
      } else {
        for (int i = 0; i < n; ++i) {
          const uint32_t t = gt + i, sbuf = t % kNBuf;
          if (PAIRS && scale2 > 0.f && i + 1 < n_ct && seg.c1 - (seg.c0 + (i + 1) * FTA_TILE) >= FTA_TILE) {
            // ---- two full cache tiles at once ------------------------------------------------
            // Everything that costs a round trip (barrier wait, TMEM load, the vote on the running
            // maximum, TMEM store, hand-off) is paid once for 128 KV rows.  The four S/P buffers let
            // the next two products be computed meanwhile.
            const uint32_t t1 = t + 1, sb1 = t1 % kNBuf;
            ok = wait_all(BAR(B_SFULL + sbuf), (t / kNBuf) & 1, abort_flag, 0x301);
            if (!ok) break;
            ok = wait_all(BAR(B_SFULL + sb1), (t1 / kNBuf) & 1, abort_flag, 0x301);
            if (!ok) break;
            if (row == 0) { FTA_TRACE(t, 3); FTA_TRACE(t1, 3); }
            tc_fence_after();
            float sa[64], sb[64];
            tmem_ld32(t_lane + kColS + FTA_TILE * sbuf, sa);
            tmem_ld32(t_lane + kColS + FTA_TILE * sbuf + 32, sa + 32);
            tmem_ld32(t_lane + kColS + FTA_TILE * sb1, sb);
            tmem_ld32(t_lane + kColS + FTA_TILE * sb1 + 32, sb + 32);
            tmem_ld_wait();
            float mx[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) mx[c] = fmax3(sa[c], sa[c + 8], sa[c + 16]);
#pragma unroll
            for (int c = 24; c + 8 < 64; c += 16)
#pragma unroll
              for (int k = 0; k < 8; ++k) mx[k] = fmax3(mx[k], sa[c + k], sa[c + 8 + k]);
#pragma unroll
            for (int c = 0; c < 64; c += 16)
#pragma unroll
              for (int k = 0; k < 8; ++k) mx[k] = fmax3(mx[k], sb[c + k], sb[c + 8 + k]);
#pragma unroll
            for (int c = 0; c < 8; ++c) mx[c] = fmaxf(mx[c], sa[56 + c]);
            const float mt = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmaxf(fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]))) * scale2;
            const bool need = mt > m_used + 8.f;
            if (i > 0 && __any_sync(0xffffffffu, need)) {
              ok = wait_all(BAR(B_ODONE + ((t - 1) & 3)), ((t - 1) >> 2) & 1, abort_flag, 0x302);
              if (!ok) break;
              tc_fence_after();
              const float alpha = need ? fta_exp2(m_used - mt) : 1.f;
#pragma unroll
              for (int ch = 0; ch < kD / 32; ++ch) {
                float o[32];
                tmem_ld32(t_lane + ch * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < 32; ++k) o[k] *= alpha;
                tmem_st32(t_lane + ch * 32, o);
              }
              tmem_st_wait();
            }
            if (need) {
              l *= fta_exp2(m_used - mt);
              m_used = mt;
            }
            const float nsub = m_used == -INFINITY ? 0.f : -m_used;
            float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const float* sv = half == 0 ? sa : sb;
              uint32_t pk[32];
#pragma unroll
              for (int c2 = 0; c2 < 32; ++c2) {
                const float2 e = ffma2(make_float2(sv[2 * c2], sv[2 * c2 + 1]), make_float2(scale2, scale2), make_float2(nsub, nsub));
                float p0, p1;
                if ((c2 & 3) == 3) { const float2 y = exp2_poly2(e); p0 = y.x; p1 = y.y; }
                else { p0 = fta_exp2(e.x); p1 = fta_exp2(e.y); }
                ps[c2 & 3] += p0 + p1;
                pk[c2] = FtaType<T>::pack(p0, p1);
              }
              const uint32_t sbh = half == 0 ? sbuf : sb1;
              if (row == 0) FTA_TRACE(half == 0 ? t : t1, 4);
              tmem_st32(t_lane + col_p(PAIRS, CS, sbh), reinterpret_cast<const float*>(pk));  // over the S columns just read
              tmem_st_wait();
              tc_fence_before();
              mbar_arrive(BAR(B_PREADY + sbh));
              if (row == 0) FTA_TRACE(half == 0 ? t : t1, 5);
            }
            l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
            ++i;  // the loop's own increment takes the second tile
            continue;
          }
          const bool is_tree = i >= n_ct;
          int valid, col0 = 0;
          if (!is_tree) {
            const int row0 = seg.c0 + i * FTA_TILE;
            valid = seg.c1 - row0 < FTA_TILE ? seg.c1 - row0 : FTA_TILE;
          } else {
            col0 = (seg.tt0 + i - n_ct) * FTA_TILE;
            valid = p.Q - col0 < FTA_TILE ? p.Q - col0 : FTA_TILE;
          }
          // a tree tile's mask row is pulled into L1 while S is still being computed
          if (is_tree && mrow != nullptr) {
#pragma unroll
            for (int c = 0; c < NC; c += 32)
              if (c < valid - cbase) asm volatile("prefetch.global.L1 [%0];" ::"l"(mrow + col0 + cbase + c));
          }
          ok = wait_all(BAR(B_SFULL + sbuf), (t / kNBuf) & 1, abort_flag, 0x301);
          if (!ok) break;
          if (row == 0) FTA_TRACE(t, 3);
          if (row == 0 && t == 0) FTA_BLK(0, clock64() - prof_t0);
          tc_fence_after();
          float s[NC];
#pragma unroll
          for (int k = 0; k < NC / 32; ++k) tmem_ld32(t_lane + kColS + FTA_TILE * sbuf + cbase + 32 * k, s + 32 * k);
          tmem_ld_wait();

          // Row maximum in the log2 domain (mt) and the factor `mul` that takes s[] there.
          // Full cache tiles keep the raw scores and fold the scale into the exponent's FMA;
          // the tree tile and the last, partial tile of a sequence take the general path.
          float mt, mul;
          if (!is_tree && valid == FTA_TILE && scale2 > 0.f) {
            float mx[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) mx[c] = fmax3(s[c], s[c + 8], s[c + 16]);
#pragma unroll
            for (int c = 24; c + 8 < NC; c += 16)
#pragma unroll
              for (int k = 0; k < 8; ++k) mx[k] = fmax3(mx[k], s[c + k], s[c + 8 + k]);
#pragma unroll
            for (int c = 0; c < 8; ++c) mx[c] = fmaxf(mx[c], s[NC - 8 + c]);
            mt = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmaxf(fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]))) * scale2;
            mul = scale2;
          } else {
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            const int vh = valid - cbase;  // valid columns among this thread's
            if (is_tree && mrow != nullptr) {
              // All loads first, so that they are in flight together; 16-byte loads where the row
              // allows it (a thread reads a row of its own, so every load costs a pass per lane).
              float mv[NC];
              const float* mp = mrow + col0 + cbase;
              const bool v4 = (reinterpret_cast<uintptr_t>(mp) & 15) == 0;
#pragma unroll
              for (int c = 0; c < NC; c += 4) {
                if (v4 && c + 3 < vh) {
                  const float4 x = __ldg(reinterpret_cast<const float4*>(mp + c));
                  mv[c] = x.x; mv[c + 1] = x.y; mv[c + 2] = x.z; mv[c + 3] = x.w;
                } else {
#pragma unroll
                  for (int k = 0; k < 4; ++k) mv[c + k] = c + k < vh ? __ldg(mp + c + k) : 0.f;
                }
              }
#pragma unroll
              for (int c = 0; c < NC; ++c) {
                float v = s[c] * scale2;
                if (c < vh) v = fmaf(mv[c], FTA_LOG2E, v);
                else v = -INFINITY;
                s[c] = v;
                mx[c & 3] = fmaxf(mx[c & 3], v);
              }
            } else {
#pragma unroll
              for (int c = 0; c < NC; ++c) {
                const float v = c < vh ? s[c] * scale2 : -INFINITY;
                s[c] = v;
                mx[c & 3] = fmaxf(mx[c & 3], v);
              }
            }
            mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            mul = 1.f;
          }
          // lazy rescale: keep the running max until it is exceeded by more than 2^8; O may only be
          // touched once the previous PV has finished
          const bool need = mt > m_used + 8.f;
          if (i > 0 && __any_sync(0xffffffffu, need)) {
            ok = wait_all(BAR(B_ODONE + ((t - 1) & 3)), ((t - 1) >> 2) & 1, abort_flag, 0x302);
            if (!ok) break;
            tc_fence_after();
            const float alpha = need ? fta_exp2(m_used - mt) : 1.f;
#pragma unroll
            for (int ch = 0; ch < kD / 32; ++ch) {
              float o[32];
              tmem_ld32(t_lane + ch * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 32; ++k) o[k] *= alpha;
              tmem_st32(t_lane + ch * 32, o);
            }
            tmem_st_wait();
          }
          if (need) {
            l *= fta_exp2(m_used - mt);
            m_used = mt;
          }
          const float nsub = m_used == -INFINITY ? 0.f : -m_used;
          float ps[4] = {0.f, 0.f, 0.f, 0.f};
          uint32_t pk[NC / 2];
#pragma unroll
          for (int c2 = 0; c2 < NC / 2; ++c2) {
            const float2 e = ffma2(make_float2(s[2 * c2], s[2 * c2 + 1]), make_float2(mul, mul), make_float2(nsub, nsub));
            // every fourth pair is exponentiated on the FMA pipe, so that the MUFU (4 lanes per
            // clock) and the FMA pipe work side by side (measured: a quarter beats a half by 1-3 %)
            float p0, p1;
            if ((c2 & 3) == 3) { const float2 y = exp2_poly2(e); p0 = y.x; p1 = y.y; }
            else { p0 = fta_exp2(e.x); p1 = fta_exp2(e.y); }
            ps[c2 & 3] += p0 + p1;
            pk[c2] = FtaType<T>::pack(p0, p1);
          }
          l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
          // P[t%3] was the A operand of PV(t-3), which completed before S(t) was even issued
          if (row == 0) FTA_TRACE(t, 4);
          if (CS == 2) tmem_st16(t_lane + col_p(PAIRS, CS, sbuf) + 16 * chalf, pk);
          else tmem_st32(t_lane + col_p(PAIRS, CS, sbuf), reinterpret_cast<const float*>(pk));  // over the S columns just read
          if (!is_tree && valid < FTA_TILE) {
            ok = zero_v_tail(t, valid);
            if (!ok) break;
          }
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(BAR(B_PREADY + sbuf));
          if (row == 0) FTA_TRACE(t, 5);
        }
        if (!ok) break;
      }

      // ---- end of the piece: the row's maximum and sum go to the epilogue warps through two
      // TMEM columns, and the next piece starts at once --------------------------------------
      if (row == 0) FTA_TRACE_EP(sidx, 0);
      ok = wait_all(BAR(B_STATSFREE), (sidx & 1) ^ 1, abort_flag, 0x307);
      if (!ok) break;
      tmem_st2(t_lane + kColStat, m_used, l);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(BAR(B_STATS));
      gt += n;
      ++sidx;
      ok = wait_all(BAR(B_SEGFULL + sidx % kSegRing), (sidx / kSegRing) & 1, abort_flag, 0x300);
      if (!ok) break;
      seg_copy(seg, &segq[sidx % kSegRing]);
      if (row == 0) FTA_TRACE_EP(sidx - 1, 1);
      if (kQBuf == 1 && seg.valid) ok = q_to_tmem(row, t_lane, sidx);
      if (row == 0) FTA_TRACE_EP(sidx - 1, 2);
    }
    if (row == 0) {
      unsigned int smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      FTA_BLK(1, clock64() - prof_t0);
      FTA_BLK(3, (long long)sidx + 1000ll * smid + 1000000ll * gt);  // pieces, SM, tiles
    }
  } else {
    // ================================ epilogue =======================================
    // O row / l and the LSE of every piece, while the softmax warps are already at work on the
    // next one.  Same row-to-thread mapping as the softmax warps (TMEM lane quadrant = warp & 3).
    reg_inc<kRegsEpilogue>();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int lrow = CS == 2 ? (row & 63) : row;
    const int chalf = CS == 2 ? (row >> 6) : 0;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
    float* ws_o = reinterpret_cast<float*>(p.workspace);
    float* ws_l = ws_o + (long long)2 * g.grid * g.R * kD;
    uint32_t gt = 0, sidx = 0, xcount = 0;
    bool ok = true;

    if (p.split_mode == FTA_SPLIT_BALANCED && row == 0)
      fta_cut_desc(p, g)[blockIdx.x] = make_int4(0, 0, 0, 0);  // rewritten below if a cut unit opens this block
    SegDesc seg, nseg;
    ok = wait_all(BAR(B_SEGFULL), 0, abort_flag, 0x500);
    if (ok) seg_copy(seg, &segq[0]);
    else seg.valid = 0;
    if (ok && seg.valid) {
      // the Q buffer goes back to the producer, for the second piece's Q, once the first is in TMEM
      if (kQBuf == 2) ok = q_to_tmem(row, t_lane, 0);
      else ok = wait_all(qready_bar(0), qready_par(0), abort_flag, 0x501);
      if (ok) mbar_arrive(BAR(B_QEMPTY));
    }
    while (ok && seg.valid) {
      FtaUnit unit;
      unit.kvh = seg.kvh; unit.gt = seg.gt; unit.qt = seg.qt;
      const int n = seg_cache_tiles(seg) + seg.tt1 - seg.tt0;
      const uint32_t t_last = gt + n - 1;
      int h, qi;
      const bool rvalid = fta_row(p, g, unit, lrow, h, qi);
      const bool working = __any_sync(0xffffffffu, rvalid) != 0;
      ok = wait_all(BAR(B_SEGFULL + (sidx + 1) % kSegRing), ((sidx + 1) / kSegRing) & 1, abort_flag, 0x500);
      if (!ok) break;
      seg_copy(nseg, &segq[(sidx + 1) % kSegRing]);
      // two Q buffers: the next piece's Q goes to TMEM as soon as it has landed, while this piece's
      // tiles are still being worked on
      if (kQBuf == 2 && nseg.valid) {
        ok = q_to_tmem(row, t_lane, sidx + 1);
        if (!ok) break;
      }

      // the row's maximum and sum, as the softmax thread of the same row left them
      ok = wait_all(BAR(B_STATS), sidx & 1, abort_flag, 0x502);
      if (!ok) break;
      tc_fence_after();
      float m_used, l;
      tmem_ld2(t_lane + kColStat, m_used, l);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(BAR(B_STATSFREE));

      ok = wait_all(BAR(B_ODONE + (t_last & 3)), (t_last >> 2) & 1, abort_flag, 0x304);
      if (!ok) break;
      tc_fence_after();
      if (row == 0) FTA_TRACE_EP(sidx, 3);

      if (!working) {
        mbar_arrive(BAR(B_OFREE));
        if (kQBuf == 1 && nseg.valid) {
          ok = wait_all(qready_bar(sidx + 1), qready_par(sidx + 1), abort_flag, 0x503);
          if (!ok) break;
        }
        if (CS == 2) {  // keep the halves' exchange barriers in step
          ok = wait_all(BAR(B_XFREE), (xcount & 1) ^ 1, abort_flag, 0x315);
          if (!ok) break;
          mbar_arrive(BAR(B_XFULL));
          mbar_arrive(BAR(B_XFREE));
          ++xcount;
        }
      } else {
        // The whole O row goes to registers at once and the accumulator is handed back: the first
        // O += P V of the next piece is waiting for exactly this.
        float o[kD];
#pragma unroll
        for (int ch = 0; ch < kD / 32; ++ch) tmem_ld32(t_lane + ch * 32, o + ch * 32);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(BAR(B_OFREE));
        if (row == 0) FTA_TRACE_EP(sidx, 4);
        // The Q buffer is this piece's staging area, but only after the next piece's Q, which has
        // been sitting in it, went to TMEM (two Q buffers: that happened above).
        if (kQBuf == 1 && nseg.valid) {
          ok = wait_all(qready_bar(sidx + 1), qready_par(sidx + 1), abort_flag, 0x503);
          if (!ok) break;
        }
        constexpr int NCOL = CS == 2 ? 64 : kD;   // output columns this thread stores
        const int col0 = CS == 2 ? 64 * chalf : 0;  // the first of them
        if (CS == 2) {
          // The two halves of the tile's rows hold two partial attentions of the same queries (over
          // the lower / upper 32 columns of every tile).  Each half parks, in shared memory, the 64
          // unnormalised O columns the OTHER half will store (16-byte chunks XOR-swizzled by row:
          // conflict-free) with its maximum and row sum, then folds what the other half parked into
          // the 64 columns it keeps: both halves merge, stage and store half a row.
          float* xo = reinterpret_cast<float*>(sm + OFF_X);  // [half that stores][row][64 columns]
          float* xm = xo + 2 * 64 * 64;                      // [half that wrote][row][m, l]
          ok = wait_all(BAR(B_XFREE), (xcount & 1) ^ 1, abort_flag, 0x30a);  // the previous piece's is read
          if (!ok) break;
          float* park = xo + ((chalf ^ 1) * 64 + lrow) * 64;
          if (chalf == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              *reinterpret_cast<float4*>(park + ((j ^ (lrow & 15)) << 2)) = make_float4(o[64 + 4 * j], o[65 + 4 * j], o[66 + 4 * j], o[67 + 4 * j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              *reinterpret_cast<float4*>(park + ((j ^ (lrow & 15)) << 2)) = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          }
          xm[(chalf * 64 + lrow) * 2] = m_used;
          xm[(chalf * 64 + lrow) * 2 + 1] = l;
          mbar_arrive(BAR(B_XFULL));
          ok = wait_all(BAR(B_XFULL), xcount & 1, abort_flag, 0x30b);
          if (!ok) break;
          const float m1 = xm[((chalf ^ 1) * 64 + lrow) * 2], l1 = xm[((chalf ^ 1) * 64 + lrow) * 2 + 1];
          const float mstar = fmaxf(m_used, m1);
          const float w0 = m_used == -INFINITY ? 0.f : fta_exp2(m_used - mstar);
          const float w1 = m1 == -INFINITY ? 0.f : fta_exp2(m1 - mstar);
          const float* mine = xo + (chalf * 64 + lrow) * 64;
          if (chalf == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float4 v = *reinterpret_cast<const float4*>(mine + ((j ^ (lrow & 15)) << 2));
              o[4 * j] = o[4 * j] * w0 + v.x * w1; o[4 * j + 1] = o[4 * j + 1] * w0 + v.y * w1;
              o[4 * j + 2] = o[4 * j + 2] * w0 + v.z * w1; o[4 * j + 3] = o[4 * j + 3] * w0 + v.w * w1;
            }
          } else {  // the kept columns 64..127 move down to o[0..63]
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float4 v = *reinterpret_cast<const float4*>(mine + ((j ^ (lrow & 15)) << 2));
              o[4 * j] = o[64 + 4 * j] * w0 + v.x * w1; o[4 * j + 1] = o[65 + 4 * j] * w0 + v.y * w1;
              o[4 * j + 2] = o[66 + 4 * j] * w0 + v.z * w1; o[4 * j + 3] = o[67 + 4 * j] * w0 + v.w * w1;
            }
          }
          l = l * w0 + l1 * w1;
          m_used = mstar;
          mbar_arrive(BAR(B_XFREE));
          ++xcount;
        }

        if (row == 0) FTA_TRACE_EP(8 + sidx, 0);
        if (p.split_mode == FTA_SPLIT_BALANCED && seg.split == 1 && row == 0)
          fta_cut_desc(p, g)[blockIdx.x] = make_int4(seg.b, seg.j, seg.nsplit, seg.p0slot);  // for stage 2
        if constexpr (CS == 1) {
          {
            const bool rstore = rvalid;
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const float lse = l > 0.f ? (m_used + fta_log2(l)) * FTA_LN2 : -INFINITY;
            const bool final_direct = p.split_mode == FTA_SPLIT_BALANCED && seg.nsplit == 1;
            const bool tree_piece = p.split_mode == FTA_SPLIT_FIXED && seg.split == g.fixed_max_splits;
            void* dst;
            int dt = FTA_DTYPE_F32;
            long long off = 0;
            if (final_direct) {
              dst = p.out; dt = p.out_dtype;
              if (rstore) {
                off = seg.b * p.o_sb + h * p.o_sh + qi * p.o_sq;
                if (p.lse) p.lse[seg.b * p.l_sb + h * p.l_sh + qi] = lse;
              }
            } else if (p.split_mode == FTA_SPLIT_BALANCED) {
              dst = ws_o; off = ((long long)seg.slot * g.R + lrow) * kD;
              if (rstore) ws_l[(long long)seg.slot * g.R + lrow] = lse;
            } else if (tree_piece) {
              dst = p.tree_o;
              if (rstore) {
                const long long ro = ((long long)seg.b * p.H + h) * p.Q + qi;
                off = ro * kD;
                p.tree_lse[ro] = lse;
              }
            } else {
              dst = p.mid_o;
              if (rstore) {
                off = seg.b * p.mo_sb + h * p.mo_sh + seg.split * p.mo_ss + qi * p.mo_sq;
                p.mid_lse[seg.b * p.ml_sb + h * p.ml_sh + seg.split * p.ml_ss + qi] = lse;
              }
            }
            // The rows go through the Q buffer, this warp's own 32 rows of it, so that every store
            // instruction of the warp writes two whole 256-byte row pieces: thread = row on the way in
            // (16-byte chunks XOR-swizzled by row), 16 lanes per row on the way out.  fp32 rows take two
            // passes of 64 columns, 16-bit rows one pass of 128.
            if (row == 0) FTA_TRACE_EP(8 + sidx, 1);
            const bool wide = dt == FTA_DTYPE_F32 ||
                              (((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && ((p.o_sb | p.o_sh | p.o_sq) & 7) == 0);
            uint8_t* stg = sm + OFF_Q;
            if (!wide) {
              if (rstore) {
  #pragma unroll
                for (int c4 = 0; c4 < kD; c4 += 4)
                  fta_store4(dst, dt, off + c4, make_float4(o[c4] * inv, o[c4 + 1] * inv, o[c4 + 2] * inv, o[c4 + 3] * inv));
              }
            } else {
              const uint32_t esize = dt == FTA_DTYPE_F32 ? 4u : 2u;
              const int c = lane & 15;
  #pragma unroll
              for (int pass = 0; pass < 2; ++pass) {
                if (pass == 1 && dt != FTA_DTYPE_F32) break;
                __syncwarp();  // the previous pass (or piece) has been read out
                if (rstore) {
  #pragma unroll
                  for (int cc = 0; cc < 16; ++cc) {
                    uint4 v;
                    if (dt == FTA_DTYPE_F32) {
                      const int e = pass * 64 + 4 * cc;
                      v.x = __float_as_uint(o[e] * inv); v.y = __float_as_uint(o[e + 1] * inv);
                      v.z = __float_as_uint(o[e + 2] * inv); v.w = __float_as_uint(o[e + 3] * inv);
                    } else if (dt == FTA_DTYPE_F16) {
                      const int e = 8 * cc;
                      v.x = FtaType<__half>::pack(o[e] * inv, o[e + 1] * inv); v.y = FtaType<__half>::pack(o[e + 2] * inv, o[e + 3] * inv);
                      v.z = FtaType<__half>::pack(o[e + 4] * inv, o[e + 5] * inv); v.w = FtaType<__half>::pack(o[e + 6] * inv, o[e + 7] * inv);
                    } else {
                      const int e = 8 * cc;
                      v.x = FtaType<__nv_bfloat16>::pack(o[e] * inv, o[e + 1] * inv); v.y = FtaType<__nv_bfloat16>::pack(o[e + 2] * inv, o[e + 3] * inv);
                      v.z = FtaType<__nv_bfloat16>::pack(o[e + 4] * inv, o[e + 5] * inv); v.w = FtaType<__nv_bfloat16>::pack(o[e + 6] * inv, o[e + 7] * inv);
                    }
                    *reinterpret_cast<uint4*>(stg + (cc >> 3) * kQHalf + row * 128 + (((cc & 7) ^ (row & 7)) << 4)) = v;
                  }
                }
                if (row == 0) FTA_TRACE_EP(8 + sidx, 2 + 3 * pass);
                __syncwarp();
                uint8_t* gdst = reinterpret_cast<uint8_t*>(dst) + pass * 256 + c * 16;
  #pragma unroll 4
                for (int it = 0; it < 16; ++it) {
                  const int rl = 2 * it + (lane >> 4);
                  const int rr = quad * 32 + rl;
                  const uint4 v = *reinterpret_cast<const uint4*>(stg + (c >> 3) * kQHalf + rr * 128 + (((c & 7) ^ (rr & 7)) << 4));
                  const long long roff = __shfl_sync(0xffffffffu, off, rl);
                  const bool rv = __shfl_sync(0xffffffffu, rstore ? 1 : 0, rl) != 0;
                  if (rv) __stcg(reinterpret_cast<uint4*>(gdst + roff * esize), v);
                }
                if (row == 0) FTA_TRACE_EP(8 + sidx, 3 + 3 * pass);
              }
              __syncwarp();
              if (row == 0) FTA_TRACE_EP(8 + sidx, 4);
            }
          }
        } else {
          {
            const bool rstore = rvalid;
            const bool lstore = rvalid && chalf == 0;  // one thread per query row writes the LSE
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const float lse = l > 0.f ? (m_used + fta_log2(l)) * FTA_LN2 : -INFINITY;
            const bool final_direct = p.split_mode == FTA_SPLIT_BALANCED && seg.nsplit == 1;
            const bool tree_piece = p.split_mode == FTA_SPLIT_FIXED && seg.split == g.fixed_max_splits;
            void* dst;
            int dt = FTA_DTYPE_F32;
            long long off = 0;
            if (final_direct) {
              dst = p.out; dt = p.out_dtype;
              if (rstore) {
                off = seg.b * p.o_sb + h * p.o_sh + qi * p.o_sq;
                if (lstore && p.lse) p.lse[seg.b * p.l_sb + h * p.l_sh + qi] = lse;
              }
            } else if (p.split_mode == FTA_SPLIT_BALANCED) {
              dst = ws_o; off = ((long long)seg.slot * g.R + lrow) * kD;
              if (lstore) ws_l[(long long)seg.slot * g.R + lrow] = lse;
            } else if (tree_piece) {
              dst = p.tree_o;
              if (rstore) {
                const long long ro = ((long long)seg.b * p.H + h) * p.Q + qi;
                off = ro * kD;
                if (lstore) p.tree_lse[ro] = lse;
              }
            } else {
              dst = p.mid_o;
              if (rstore) {
                off = seg.b * p.mo_sb + h * p.mo_sh + seg.split * p.mo_ss + qi * p.mo_sq;
                if (lstore) p.mid_lse[seg.b * p.ml_sb + h * p.ml_sh + seg.split * p.ml_ss + qi] = lse;
              }
            }
            off += col0;
            // The row slices go through the Q buffer, each thread's own 128-byte lines of it, so that
            // every store instruction of the warp writes whole row slices: thread = row on the way in
            // (16-byte chunks XOR-swizzled by row), 8 or 16 lanes per row on the way out.  A pass moves
            // up to 256 bytes per row; only full fp32 rows (512 bytes) take two.
            if (row == 0) FTA_TRACE_EP(8 + sidx, 1);
            const bool wide = dt == FTA_DTYPE_F32 ||
                              (((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && ((p.o_sb | p.o_sh | p.o_sq) & 7) == 0);
            uint8_t* stg = sm + OFF_Q;
            if (!wide) {
              if (rstore) {
  #pragma unroll
                for (int c4 = 0; c4 < NCOL; c4 += 4)
                  fta_store4(dst, dt, off + c4, make_float4(o[c4] * inv, o[c4 + 1] * inv, o[c4 + 2] * inv, o[c4 + 3] * inv));
              }
            } else {
              const uint32_t esize = dt == FTA_DTYPE_F32 ? 4u : 2u;
              const uint32_t slice = NCOL * esize;                 // bytes of a row this thread stores
              const uint32_t pbytes = slice < 256u ? slice : 256u;  // per pass
              const int npass = (int)(slice / pbytes);
              const int lpr = CS == 1 ? 16 : (int)(pbytes / 16u);  // 16-byte chunks = lanes per row
              const int c = lane & (lpr - 1), rsub = lane / lpr, rpi = 32 / lpr;
  #pragma unroll
              for (int pass = 0; pass < 2; ++pass) {
                if (pass >= npass) break;
                __syncwarp();  // the previous pass (or piece) has been read out
                if (rstore) {
  #pragma unroll
                  for (int cc = 0; cc < 16; ++cc) {
                    if (CS == 2 && cc >= lpr) break;
                    uint4 v;
                    if (dt == FTA_DTYPE_F32) {
                      const int e = (pass * 64 + 4 * cc) % NCOL;
                      v.x = __float_as_uint(o[e] * inv); v.y = __float_as_uint(o[e + 1] * inv);
                      v.z = __float_as_uint(o[e + 2] * inv); v.w = __float_as_uint(o[e + 3] * inv);
                    } else if (dt == FTA_DTYPE_F16) {
                      const int e = (8 * cc) % NCOL;
                      v.x = FtaType<__half>::pack(o[e] * inv, o[e + 1] * inv); v.y = FtaType<__half>::pack(o[e + 2] * inv, o[e + 3] * inv);
                      v.z = FtaType<__half>::pack(o[e + 4] * inv, o[e + 5] * inv); v.w = FtaType<__half>::pack(o[e + 6] * inv, o[e + 7] * inv);
                    } else {
                      const int e = (8 * cc) % NCOL;
                      v.x = FtaType<__nv_bfloat16>::pack(o[e] * inv, o[e + 1] * inv); v.y = FtaType<__nv_bfloat16>::pack(o[e + 2] * inv, o[e + 3] * inv);
                      v.z = FtaType<__nv_bfloat16>::pack(o[e + 4] * inv, o[e + 5] * inv); v.w = FtaType<__nv_bfloat16>::pack(o[e + 6] * inv, o[e + 7] * inv);
                    }
                    *reinterpret_cast<uint4*>(stg + (cc >> 3) * kQHalf + row * 128 + (((cc & 7) ^ (row & 7)) << 4)) = v;
                  }
                }
                if (row == 0) FTA_TRACE_EP(8 + sidx, 2 + 3 * pass);
                __syncwarp();
                uint8_t* gdst = reinterpret_cast<uint8_t*>(dst) + pass * 256 + c * 16;
  #pragma unroll 4
                for (int it = 0; it < 16; ++it) {
                  if (CS == 2 && it >= lpr) break;  // 32 rows, 32 / lpr of them per instruction
                  const int rl = it * rpi + rsub;
                  const int rr = quad * 32 + rl;
                  const uint4 v = *reinterpret_cast<const uint4*>(stg + (c >> 3) * kQHalf + rr * 128 + (((c & 7) ^ (rr & 7)) << 4));
                  const long long roff = __shfl_sync(0xffffffffu, off, rl);
                  const bool rv = __shfl_sync(0xffffffffu, rstore ? 1 : 0, rl) != 0;
                  if (rv) __stcg(reinterpret_cast<uint4*>(gdst + roff * esize), v);
                }
                if (row == 0) FTA_TRACE_EP(8 + sidx, 3 + 3 * pass);
              }
              __syncwarp();
              if (row == 0) FTA_TRACE_EP(8 + sidx, 4);
            }
          }
        }
      }
      if (row == 0) FTA_TRACE_EP(sidx, 6);
      if (nseg.valid) {  // the staging area is the Q buffer of the piece after next again
        fence_proxy_async();
        mbar_arrive(BAR(B_QEMPTY));
      }
      if (lane == 0) mbar_arrive(BAR(B_SEGFREE + sidx % kSegRing));
      gt += n;
      ++sidx;
      seg = nseg;
    }
    if (row == 0) FTA_BLK(2, clock64() - prof_t0);
  }

#ifdef FTA_UMMA_PROFILE
  if (tid == 0) {
    unsigned long long gt1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt1));
    if (blockIdx.x == 0) atomicAdd(&g_umma_prof[159], (unsigned long long)(clock64() - prof_t0));
    atomicMax(&g_umma_prof[158], (unsigned long long)(clock64() - prof_t0));
    atomicMax(&g_umma_prof[157], gt1 - prof_g0);
  }
#endif
  // ---- teardown -------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
#undef BAR
}

// ---- host side: tensor maps --------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

struct MapKey {
  const void* ptr;
  int dtype;
  uint64_t dims[5];
  int64_t strides[4];
  uint32_t box[5];
  bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kMapCache = 64;
MapEntry g_maps[kMapCache];
int g_map_next = 0;
std::mutex g_map_mu;

// Map over a [B, heads, rows, 128] tensor with element strides (rows, heads, batch); boxes of 64
// columns (one 128-byte swizzle span) x box_rows x box_heads, zero fill out of bounds.
//   both_halves: 5-D, the two halves of the 128 columns are a dimension of their own placed after
//                the heads, so that ONE copy lands as [half][row][64 columns] (K and V tiles: the
//                second half starts box_rows * 128 bytes after the first);
//   otherwise:   4-D, one copy per half (the Q tile, whose halves sit 128 rows apart whatever the
//                number of rows the box has).
bool make_map(CUtensorMap* out, const void* ptr, int dtype, uint64_t rows, uint64_t heads, uint64_t B, int64_t s_row,
              int64_t s_head, int64_t s_batch, uint32_t box_rows, uint32_t box_heads, bool both_halves) {
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.ptr = ptr; key.dtype = dtype;
  key.dims[0] = both_halves ? 64 : kD; key.dims[1] = rows; key.dims[2] = heads; key.dims[3] = both_halves ? 2 : 1; key.dims[4] = B;
  // a stride of a size-1 dimension is never used; give it a value the encoder accepts
  if (heads == 1) s_head = s_row * (int64_t)rows;
  if (B == 1) s_batch = s_head * (int64_t)heads;
  if (rows == 1) s_row = kD;
  key.strides[0] = s_row; key.strides[1] = s_head; key.strides[2] = 64; key.strides[3] = s_batch;
  key.box[0] = 64; key.box[1] = box_rows; key.box[2] = box_heads; key.box[3] = both_halves ? 2 : 1; key.box[4] = 1;
  std::lock_guard<std::mutex> lock(g_map_mu);
  for (int i = 0; i < kMapCache; ++i)
    if (g_maps[i].used && g_maps[i].key == key) { *out = g_maps[i].map; return true; }
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t gdim[5] = {key.dims[0], key.dims[1], key.dims[2], key.dims[3], key.dims[4]};
  cuuint64_t gstr[4] = {(cuuint64_t)s_row * 2, (cuuint64_t)s_head * 2, 128, (cuuint64_t)s_batch * 2};
  cuuint32_t box[5] = {key.box[0], key.box[1], key.box[2], key.box[3], key.box[4]};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMap m;
  const CUtensorMapDataType dt = dtype == FTA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r;
  if (both_halves) {
    r = enc(&m, dt, 5, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    // 4-D: {128 columns, rows, heads, batch}, box of 64 columns; the caller loads the halves one by one
    cuuint64_t gdim4[4] = {(cuuint64_t)kD, key.dims[1], key.dims[2], key.dims[4]};
    cuuint64_t gstr4[3] = {(cuuint64_t)s_row * 2, (cuuint64_t)s_head * 2, (cuuint64_t)s_batch * 2};
    cuuint32_t box4[4] = {64, box_rows, box_heads, 1};
    r = enc(&m, dt, 4, const_cast<void*>(ptr), gdim4, gstr4, box4, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return false;
  MapEntry& e = g_maps[g_map_next];
  g_map_next = (g_map_next + 1) % kMapCache;
  e.key = key; e.map = m; e.used = true;
  *out = m;
  return true;
}

bool stride_ok(int64_t s) { return s > 0 && s % 8 == 0 && s * 2 < (1ll << 40); }

}  // namespace fta_umma

using namespace fta_umma;

// The tcgen05 family serves head_dim 128 with positive 16-byte-multiple strides.
int fta_umma_supported(const FtaParams& p) {
  if (p.D != kD || p.ctx < 1 || p.B < 1) return 0;
  if (!stride_ok(p.q_sq) || !stride_ok(p.k_st) || !stride_ok(p.v_st)) return 0;
  if (p.H > 1 && !stride_ok(p.q_sh)) return 0;
  if (p.Hkv > 1 && (!stride_ok(p.k_sh) || !stride_ok(p.v_sh))) return 0;
  if (p.B > 1 && !stride_ok(p.q_sb)) return 0;
  if ((p.block_table ? p.n_pages : p.B) > 1 && (!stride_ok(p.k_sb) || !stride_ok(p.v_sb))) return 0;
  if (p.with_tree) {
    if (!stride_ok(p.ck_st) || !stride_ok(p.cv_st)) return 0;
    if (p.Hkv * p.cur_head_mul > 1 && (!stride_ok(p.ck_sh) || !stride_ok(p.cv_sh))) return 0;
    if (p.B > 1 && (!stride_ok(p.ck_sb) || !stride_ok(p.cv_sb))) return 0;
  }
  // the block's shared memory (prefix table of B + 1 entries included) must fit with five stages
  const int G = p.H / p.Hkv;
  const int qpt = p.Q < kR ? p.Q : kR;
  const int hpt = kR / qpt < G ? kR / qpt : G;
  if (smem_bytes(5, p.B, hpt * qpt <= 64 ? 2 : 1) > 227 * 1024) return 0;
  return get_encode() != nullptr ? 1 : 0;
}

cudaError_t fta_launch_stage1_umma(const FtaParams& p, const FtaGeom& g, cudaStream_t st, int query_only,
                                   int* blocks_per_sm, int overlap) {
  // six ring stages when everything else leaves room for them, else five
  const int cs = g.cs == 2 ? 2 : 1;
  const int ns = smem_bytes(6, p.B, cs) <= 227 * 1024 ? 6 : 5;
  const size_t smem = smem_bytes(ns, p.B, cs);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  void (*kern)(const FtaParams, const FtaGeom, const Maps);
  const bool f16 = p.dtype == FTA_DTYPE_F16;
  // Tiles are taken two at a time (and a fourth S/P buffer is used) only where the blocks are fed
  // through L2: several M tiles per KV head walking the same tiles (lanes).  Where every block streams
  // its own K/V from DRAM, letting the products and the softmax run further ahead makes the blocks
  // compete for memory unevenly and the slowest one ends later (measured on cfg 3: +8 %).
  const bool pairs = cs == 1 && g.lanes > 1;
  if (cs == 2) {
    if (f16) kern = ns == 6 ? stage1_umma_kernel<__half, 6, 2, false> : stage1_umma_kernel<__half, 5, 2, false>;
    else kern = ns == 6 ? stage1_umma_kernel<__nv_bfloat16, 6, 2, false> : stage1_umma_kernel<__nv_bfloat16, 5, 2, false>;
  } else if (pairs) {
    if (f16) kern = ns == 6 ? stage1_umma_kernel<__half, 6, 1, true> : stage1_umma_kernel<__half, 5, 1, true>;
    else kern = ns == 6 ? stage1_umma_kernel<__nv_bfloat16, 6, 1, true> : stage1_umma_kernel<__nv_bfloat16, 5, 1, true>;
  } else {
    if (f16) kern = ns == 6 ? stage1_umma_kernel<__half, 6, 1, false> : stage1_umma_kernel<__half, 5, 1, false>;
    else kern = ns == 6 ? stage1_umma_kernel<__nv_bfloat16, 6, 1, false> : stage1_umma_kernel<__nv_bfloat16, 5, 1, false>;
  }
  static unsigned long long configured[12] = {0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const int ti = (f16 ? 0 : 1) + (ns == 6 ? 0 : 2) + (cs == 2 ? 4 : (pairs ? 8 : 0));
  if (!((configured[ti] >> (dev & 63)) & 1ull)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    configured[ti] |= 1ull << (dev & 63);
  }
  if (query_only) return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, kern, kThreads, smem);

  Maps maps;
  const int Hcur = p.Hkv * p.cur_head_mul;
  // the cache as the copy engine sees it: [B, Hkv, ctx, D], or a pool of pages [n_pages, Hkv, page_size, D]
  const uint64_t crows = p.block_table ? (uint64_t)p.page_size : (uint64_t)p.ctx;
  const uint64_t cbatch = p.block_table ? (uint64_t)p.n_pages : (uint64_t)p.B;
  bool ok = make_map(&maps.q, p.q, p.dtype, p.Q, p.H, p.B, p.q_sq, p.q_sh, p.q_sb, g.qpt, g.hpt, false) &&
            make_map(&maps.k, p.k_cache, p.dtype, crows, p.Hkv, cbatch, p.k_st, p.k_sh, p.k_sb, FTA_TILE, 1, true) &&
            make_map(&maps.v, p.v_cache, p.dtype, crows, p.Hkv, cbatch, p.v_st, p.v_sh, p.v_sb, FTA_TILE, 1, true);
  if (ok && p.with_tree) {
    ok = make_map(&maps.ck, p.cur_k, p.dtype, p.Q, Hcur, p.B, p.ck_st, p.ck_sh, p.ck_sb, FTA_TILE, 1, true) &&
         make_map(&maps.cv, p.cur_v, p.dtype, p.Q, Hcur, p.B, p.cv_st, p.cv_sh, p.cv_sb, FTA_TILE, 1, true);
  } else if (ok) {
    maps.ck = maps.k;
    maps.cv = maps.v;
  }
  if (!ok) return cudaErrorInvalidValue;
  // overlap: with programmatic stream serialization the blocks are placed and set themselves up
  // (barriers, tensor memory, descriptors) while the kernel before this one in the stream drains, if
  // that kernel allows it (the previous call's stage 2 does); they touch global memory only after
  // griddepcontrol.wait.  After any other kernel the launch behaves like an ordinary one.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g.grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cfg.attrs = attr; cfg.numAttrs = overlap ? 1 : 0;
  const cudaError_t e2 = cudaLaunchKernelEx(&cfg, kern, p, g, maps);
  return e2 != cudaSuccess ? e2 : cudaGetLastError();
}

#ifdef FTA_UMMA_PROFILE
extern "C" int fta_umma_trace(long long* out512) {
  return cudaMemcpyFromSymbol(out512, g_umma_trace, sizeof(long long) * 640) == cudaSuccess ? 0 : -1;
}
extern "C" int fta_umma_blocks(long long* out4096) {
  return cudaMemcpyFromSymbol(out4096, g_umma_blk, sizeof(long long) * 4096) == cudaSuccess ? 0 : -1;
}
extern "C" int fta_umma_prof(unsigned long long* out64) {
  unsigned long long zero[160] = {0};
  if (cudaMemcpyFromSymbol(out64, g_umma_prof, sizeof(zero)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(g_umma_prof, zero, sizeof(zero));
  return 0;
}
#endif

// Reads and clears the device status word: 0, or the code of the first bounded wait that gave up.
extern "C" int fta_umma_status(void) {
  unsigned int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(v)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(zero));
  return (int)v;
}
