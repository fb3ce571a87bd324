// Stage 2: log-sum-exp merge of the partial attentions stage 1 left behind, one warp
// per query row, float4 along head_dim.
//
// It replaces the reference's _flash_decoding_fwd_reduce_kernel (flash_tree_attn.py:146-211)
// and the final two-way blend with the tree part (flash_tree_attn.py:373).  The recurrence
// is the reference's (:195-208): m' = max(m, lse_s); acc = acc*e^(m-m') + e^(lse_s-m')*o_s;
// l = l*e^(m-m') + e^(lse_s-m').  Unlike the reference the LSE stays fp32 throughout (the
// reference rounds it to the query dtype, :285,:211, before the blend).
#include "fta_common.cuh"

namespace {

struct Acc {
  float m, l;
  float4 a;
  __device__ __forceinline__ void init() { m = -INFINITY; l = 0.f; a = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void add(float lse, const float4& o) {
    if (lse == -INFINITY) return;  // an empty partial contributes nothing
    const float mn = fmaxf(m, lse);
    const float sc = __expf(m - mn);  // m == -inf -> 0
    const float w = __expf(lse - mn);
    a.x = a.x * sc + w * o.x; a.y = a.y * sc + w * o.y;
    a.z = a.z * sc + w * o.z; a.w = a.w * sc + w * o.w;
    l = l * sc + w;
    m = mn;
  }
  __device__ __forceinline__ float4 value() const {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    return make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
  }
  __device__ __forceinline__ float lse() const { return l > 0.f ? m + __logf(l) : -INFINITY; }
};

constexpr int kThreads = 256;
constexpr int kRowsPerWarp = 2;  // BALANCED: two rows in flight per warp, and the whole merge fits one wave of blocks
constexpr int kRowsPerBlock = kThreads / 32;

// Waits until the kernel launched before this one on the stream (stage 1) has completed and its
// stores are visible.  Stage 2 is launched with programmatic stream serialization, so its blocks are
// set up while stage 1 still runs and start the moment it has finished.
// Also lets a kernel that follows in the stream and was launched the same way (the next call's stage 1)
// be set up now; it reads and writes nothing before its own griddepcontrol.wait, which returns once
// this grid, and so the stage 1 it waited for, has finished.
__device__ __forceinline__ void wait_for_stage1() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// One warp per query row (two rows per warp in the BALANCED plan), one float4 of head_dim per lane (two
// for head_dim 256).  Loads of up to four partials per row are issued before any is folded in.
//   BALANCED: grid = (stage-1 blocks, row groups): block c merges the unit whose second piece
//             opens stage-1 block c, if any (fta_cut_desc); uncut units were finished by stage 1.
//   FIXED:    grid = (units, row groups).
__global__ void __launch_bounds__(kThreads) stage2_kernel(const FtaParams p, const FtaGeom g, const int ask_first) {
  const int lane = threadIdx.x & 31;
  const int D = p.D;
  wait_for_stage1();

  if (p.split_mode == FTA_SPLIT_BALANCED) {
    const int row0 = (blockIdx.y * kRowsPerBlock + (threadIdx.x >> 5)) * kRowsPerWarp;
    if (row0 >= g.R) return;
    const float* ws_o = reinterpret_cast<const float*>(p.workspace);
    const float* ws_l = ws_o + (long long)2 * g.grid * g.R * D;
    // Every piece of the unit this block may have to merge sits in a slot that follows from the block
    // index alone (piece 0: slot 1 of block - lanes, the block that walked the range before this one's
    // for the same M tile; piece i >= 1: slot 0 of block + (i - 1) * lanes), so the loads of pieces 0
    // and 1 go out together with the load of the cut descriptor (which says whether there is anything
    // to merge and how many pieces): a round trip less on a path that is nothing but round trips.  A
    // slot read in vain is inside the workspace.
    // Piece 1's slot is this block's own and is always asked for; piece 0's only where most blocks
    // do merge (ask_first: at least as many units as blocks, so a unit is cut once at most) - with few
    // long units most blocks open with a third or later piece and would read it in vain.
    constexpr int kAhead = 2;  // pieces 0 and 1: both needed whenever there is anything to merge
    const int c40 = lane * 4;
    float lse_a[kRowsPerWarp][kAhead];
    float4 o_a[kRowsPerWarp][kAhead];
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      const long long slot = k == 0 ? 2ll * ((long long)blockIdx.x - g.lanes) + 1 : 2ll * (long long)blockIdx.x;
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        lse_a[r][k] = -INFINITY; o_a[r][k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (slot >= 0 && (k > 0 || ask_first) && row0 + r < g.R && c40 < D) {
          lse_a[r][k] = ws_l[slot * g.R + row0 + r];
          o_a[r][k] = *reinterpret_cast<const float4*>(ws_o + (slot * g.R + row0 + r) * D + c40);
        }
      }
    }
    const int4 cut = fta_cut_desc(p, g)[blockIdx.x];
    const int np = cut.z;
    if (np < 2) return;
    const int b = cut.x, j = cut.y;
    const FtaUnit unit = fta_unit(g, j);
    int h[kRowsPerWarp], qi[kRowsPerWarp];
    bool live[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) live[r] = row0 + r < g.R && fta_row(p, g, unit, row0 + r, h[r], qi[r]);
    for (int c4 = c40; c4 < D; c4 += 128) {
      Acc acc[kRowsPerWarp];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) acc[r].init();
      // pieces in order: 0 and 1 (already here for the first 128 columns), then the rest four at a time
      if (c4 == c40 && ask_first) {
#pragma unroll
        for (int k = 0; k < kAhead; ++k)
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r)
            if (live[r]) acc[r].add(lse_a[r][k], o_a[r][k]);
      } else {
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
          if (!live[r]) continue;
          const long long slot = cut.w;
          acc[r].add(ws_l[slot * g.R + row0 + r], *reinterpret_cast<const float4*>(ws_o + (slot * g.R + row0 + r) * D + c4));
        }
        if (c4 == c40) {
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r)
            if (live[r]) acc[r].add(lse_a[r][1], o_a[r][1]);
        }
      }
      for (int s0 = c4 == c40 ? kAhead : 1; s0 < np; s0 += 4) {
        float lse[kRowsPerWarp][4]; float4 o[kRowsPerWarp][4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int s = s0 + k;
          const long long slot = 2ll * ((long long)blockIdx.x + (long long)(s - 1) * g.lanes);
#pragma unroll
          for (int r = 0; r < kRowsPerWarp; ++r) {
            lse[r][k] = -INFINITY; o[r][k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s < np && live[r]) {
              lse[r][k] = ws_l[slot * g.R + row0 + r];
              o[r][k] = *reinterpret_cast<const float4*>(ws_o + (slot * g.R + row0 + r) * D + c4);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[r].add(lse[r][k], o[r][k]);
      }
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        if (!live[r]) continue;
        fta_store4(p.out, p.out_dtype, b * p.o_sb + h[r] * p.o_sh + qi[r] * p.o_sq + c4, acc[r].value());
        if (c4 == 0 && p.lse) p.lse[b * p.l_sb + h[r] * p.l_sh + qi[r]] = acc[r].lse();
      }
    }
    return;
  }

  const int row = blockIdx.y * kRowsPerBlock + (threadIdx.x >> 5);
  if (row >= g.R) return;
  const int b = blockIdx.x / g.U, j = blockIdx.x - b * g.U;
  const FtaUnit unit = fta_unit(g, j);
  int h, qi;
  if (!fta_row(p, g, unit, row, h, qi)) return;
  // FIXED: cache partials in mid_o/mid_lse, the tree partial in tree_o/tree_lse
  const int Lb = fta_load_len(p.kv_seq_len, p.len_is_i64, b, p.ctx);
  const int np = fta_cdiv(Lb, p.split_tokens);
  for (int c4 = lane * 4; c4 < D; c4 += 128) {
    Acc acc; acc.init();
    const float* mo = p.mid_o + b * p.mo_sb + h * p.mo_sh + qi * p.mo_sq + c4;
    const float* ml = p.mid_lse + b * p.ml_sb + h * p.ml_sh + qi;
    for (int s0 = 0; s0 < np; s0 += 4) {
      float lse[4]; float4 o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int s = s0 + k;
        lse[k] = -INFINITY; o[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (s < np) {
          lse[k] = ml[s * p.ml_ss];
          o[k] = *reinterpret_cast<const float4*>(mo + s * p.mo_ss);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) acc.add(lse[k], o[k]);
    }
    if (p.out_cache)
      fta_store4(p.out_cache, p.dtype, b * p.oc_sb + h * p.oc_sh + qi * p.oc_sq + c4, acc.value());
    if (g.n_tree > 0) {
      const long long ro = ((long long)b * p.H + h) * p.Q + qi;
      acc.add(p.tree_lse[ro], *reinterpret_cast<const float4*>(p.tree_o + ro * D + c4));
    }
    fta_store4(p.out, p.out_dtype, b * p.o_sb + h * p.o_sh + qi * p.o_sq + c4, acc.value());
    if (c4 == 0 && p.lse) p.lse[b * p.l_sb + h * p.l_sh + qi] = acc.lse();
  }
}

// BALANCED without the tree tokens: a sequence of length 0 has no tile at all, so no stage-1 block
// ever writes its rows; they are defined here (zero output, LSE = -inf).
__global__ void __launch_bounds__(kThreads) empty_rows_kernel(const FtaParams p) {
  const int b = blockIdx.x;
  wait_for_stage1();
  if (fta_load_len(p.kv_seq_len, p.len_is_i64, b, p.ctx) != 0) return;
  const int D4 = p.D >> 2;
  for (int i = threadIdx.x; i < p.H * p.Q * D4; i += kThreads) {
    const int c4 = (i % D4) * 4, hq = i / D4, qi = hq % p.Q, h = hq / p.Q;
    fta_store4(p.out, p.out_dtype, b * p.o_sb + h * p.o_sh + qi * p.o_sq + c4, make_float4(0.f, 0.f, 0.f, 0.f));
    if (c4 == 0 && p.lse) p.lse[b * p.l_sb + h * p.l_sh + qi] = -INFINITY;
  }
}

__global__ void __launch_bounds__(kThreads) merge_parts_kernel(const FtaMergeParams p) {
  const int D4 = p.D >> 2;
  const long long n = (long long)p.rows * D4;
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads) {
    const long long row = i / D4;
    const int c4 = (int)(i - row * D4) * 4;
    Acc acc; acc.init();
    for (int s = 0; s < p.n_parts; ++s)
      acc.add(p.part_lse[s * p.pl_ss + row],
              *reinterpret_cast<const float4*>(p.part_o + s * p.po_ss + row * p.D + c4));
    fta_store4(p.out, p.out_dtype, row * p.D + c4, acc.value());
    if (c4 == 0 && p.lse) p.lse[row] = acc.lse();
  }
}

// ---- exchange + merge for KV-range shards on several GPUs ------------------------------------
// Every rank keeps its packed partial ([rows, D] O then [rows] LSE, fp32) in memory its peers have
// mapped.  One launch per rank: block 0 tells every peer "my partial of call `epoch` is complete"
// with a release store into the peer's flag array, every block waits until each peer has said the
// same (acquire loads of this rank's own flag array, bounded by a timeout), then the merge reads
// the peers' partials with plain loads over NVLink and folds them in rank order.
//   * The partial was written by earlier kernels on this stream, so it is complete when this kernel
//     starts; the peers read it where it lives (pull), so no data has to be ordered after a flag.
//   * Flags only grow (the epoch of the last finished call), so nothing is ever reset.
//   * A rank rewrites a buffer two calls later.  A peer that still reads the buffer of call e has
//     not yet signalled e + 1, and this rank's call e + 1 waits for that signal before it ends, so
//     two alternating buffers are enough.
//   * When a wait runs out the block leaves without storing and sets *status; the host reads it.
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Threads 0..world-1 of the block except this rank's own (one per peer): tell the peer (when `signal`) and wait until the
// peer has told us; `slot` selects the first or the second flag round.  Returns through *fail a
// bit per peer whose signal did not come within the limit.
__device__ __forceinline__ void exchange_round(const FtaExchangeParams& p, int slot, bool signal, int* fail) {
  const int t = threadIdx.x;
  if (t < p.world && t != p.rank) {
    if (signal) {
      __threadfence_system();
      st_release_sys(p.flag_peer[t] + slot * p.world, p.epoch);
    }
    const unsigned* mine = p.flag_local + slot * p.world + t;
    const unsigned long long t0 = global_ns();
    unsigned spins = 0;
    while ((int)(ld_acquire_sys(mine) - p.epoch) < 0) {
      if ((++spins & 31u) == 0 && global_ns() - t0 > (unsigned long long)p.timeout_ns) {
        atomicOr(fail, 1 << (t + 8 * slot));
        break;
      }
      __nanosleep(32);
    }
  }
}

// Folds rank 0..world-1's partials of one float4 of one row, in rank order.
__device__ __forceinline__ Acc exchange_fold(const FtaExchangeParams& p, long long row, int c4) {
  const long long lse_off = (long long)p.rows * p.D;
  float lse[FTA_MAX_RANKS];
  float4 o[FTA_MAX_RANKS];
#pragma unroll
  for (int s = 0; s < FTA_MAX_RANKS; ++s)
    if (s < p.world) {
      lse[s] = __ldcg(p.part[s] + lse_off + row);
      o[s] = __ldcg(reinterpret_cast<const float4*>(p.part[s] + row * p.D + c4));
    }
  Acc acc; acc.init();
#pragma unroll
  for (int s = 0; s < FTA_MAX_RANKS; ++s)
    if (s < p.world) acc.add(lse[s], o[s]);
  return acc;
}

// Every rank reads every peer's whole partial and merges all rows itself: one flag round.
__global__ void __launch_bounds__(kThreads) exchange_merge_kernel(const FtaExchangeParams p) {
  __shared__ int s_fail;
  const int t = threadIdx.x;
  if (t == 0) s_fail = 0;
  __syncthreads();
  exchange_round(p, 0, blockIdx.x == 0, &s_fail);
  __syncthreads();
  if (s_fail) {
    if (t == 0) atomicOr(p.status, s_fail);
    return;
  }
  const int D4 = p.D >> 2;
  const long long n = (long long)p.rows * D4;
  for (long long i = (long long)blockIdx.x * kThreads + t; i < n; i += (long long)gridDim.x * kThreads) {
    const long long row = i / D4;
    const int c4 = (int)(i - row * D4) * 4;
    const Acc acc = exchange_fold(p, row, c4);
    fta_store4(p.out, p.out_dtype, row * p.D + c4, acc.value());
    if (c4 == 0 && p.lse) p.lse[row] = acc.lse();
  }
}

// With many ranks reading everything from everybody is an all-gather of the fp32 partials
// ((world - 1) x the partial over NVLink into every GPU).  Here each rank merges only ITS slice of
// the rows (reads 1/world of every peer's partial) and stores the merged, rounded rows into every
// rank's result buffer (peer-mapped as well): about (world - 1) / world of ONE partial in and half
// of that out per GPU.  Two flag rounds: "my partial is ready", then, from the last block to finish
// its stores, "my slice is in your result buffer"; the kernel ends when every peer's slice is in.
//   * Nobody stores into a peer's result buffer before that peer has signalled the first round of
//     this call, i.e. before the peer's stream has passed everything that read the previous result.
//   * p.done[0] counts finished blocks and p.done[1] collects the waits that ran out in THIS launch;
//     the last block sets both back to zero.  The second round is skipped when this launch lost a
//     wait, whatever an earlier launch left in *p.status (which stays set until the host reads it).
__global__ void __launch_bounds__(kThreads) exchange_scatter_kernel(const FtaExchangeParams p) {
  __shared__ int s_fail, s_last;
  const int t = threadIdx.x;
  if (t == 0) s_fail = 0;
  __syncthreads();
  exchange_round(p, 0, blockIdx.x == 0, &s_fail);
  __syncthreads();
  if (s_fail) {
    if (t == 0) {
      atomicOr(p.status, s_fail);
      atomicOr(p.done + 1, s_fail);
    }
  } else {
    const int D4 = p.D >> 2;
    const int per = (p.rows + p.world - 1) / p.world;
    const int r0 = min(p.rows, p.rank * per), r1 = min(p.rows, r0 + per);
    const long long n = (long long)(r1 - r0) * D4;
    for (long long i = (long long)blockIdx.x * kThreads + t; i < n; i += (long long)gridDim.x * kThreads) {
      const long long row = r0 + i / D4;
      const int c4 = (int)(i % D4) * 4;
      const Acc acc = exchange_fold(p, row, c4);
      const float4 v = acc.value();
      const float l = acc.lse();
#pragma unroll
      for (int s = 0; s < FTA_MAX_RANKS; ++s)
        if (s < p.world) {
          fta_store4(p.out_peer[s], p.out_dtype, row * p.D + c4, v);
          if (c4 == 0) p.lse_peer[s][row] = l;
        }
    }
  }
  // One system-scope fence per block, after the barrier that makes the block's stores visible to
  // thread 0 (a fence in every warp costs an NVLink round trip each and they queue up per SM).
  __syncthreads();
  if (t == 0) {
    __threadfence_system();
    s_last = atomicAdd(p.done, 1) == (int)gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  if (t == 0) {
    s_fail = *reinterpret_cast<volatile int*>(p.done + 1);  // some block of this launch gave up: no second round
    p.done[0] = 0;
    p.done[1] = 0;
  }
  __syncthreads();
  if (s_fail) return;
  exchange_round(p, 1, true, &s_fail);
  __syncthreads();
  if (t == 0 && s_fail) atomicOr(p.status, s_fail);
}

}  // namespace

cudaError_t fta_launch_exchange_merge(const FtaExchangeParams& p, cudaStream_t st) {
  const bool scatter = p.done != nullptr;
  const long long rows = scatter ? (p.rows + p.world - 1) / p.world : p.rows;
  const long long n = rows * (p.D >> 2);
  long long blocks = (n + kThreads - 1) / kThreads;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  if (scatter)
    exchange_scatter_kernel<<<(int)blocks, kThreads, 0, st>>>(p);
  else
    exchange_merge_kernel<<<(int)blocks, kThreads, 0, st>>>(p);
  return cudaGetLastError();
}

cudaError_t fta_launch_stage2(const FtaParams& p, const FtaGeom& g, cudaStream_t st, int overlap) {
  const bool balanced = p.split_mode == FTA_SPLIT_BALANCED;
  // rows past hpt * qpt of a unit's tile are padding: no blocks for them
  const int rows = g.hpt * g.qpt < g.R ? g.hpt * g.qpt : g.R;
  const int rpb = kRowsPerBlock * (balanced ? kRowsPerWarp : 1);
  const dim3 grid(balanced ? g.grid : p.B * g.U, (rows + rpb - 1) / rpb);
  // Programmatic stream serialization: the grid is set up while stage 1 is still running and its
  // blocks wait (griddepcontrol.wait) for stage 1 to finish, instead of being launched after it.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = 0; cfg.stream = st;
  cfg.attrs = attr; cfg.numAttrs = overlap ? 1 : 0;  // 0: an ordinary launch (the stage is being timed alone)
  // units on the line against groups of blocks that share it
  const int ask_first = balanced && (long long)p.B * g.U >= (long long)g.grid ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, stage2_kernel, p, g, ask_first);
  if (e != cudaSuccess) return e;
  if (balanced && !p.with_tree) {
    cfg.gridDim = dim3(p.B);
    e = cudaLaunchKernelEx(&cfg, empty_rows_kernel, p);
    if (e != cudaSuccess) return e;
  }
  return cudaGetLastError();
}

cudaError_t fta_launch_merge_parts(const FtaMergeParams& p, cudaStream_t st) {
  const long long n = (long long)p.rows * (p.D >> 2);
  long long blocks = (n + kThreads - 1) / kThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  merge_parts_kernel<<<(int)blocks, kThreads, 0, st>>>(p);
  return cudaGetLastError();
}
