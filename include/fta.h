/*
 * fta.h — C ABI of the B200 tree-attention decode library (libfta.so).
 *
 * One operator is exported: the tree-attention verification step of speculative
 * decoding.  Q tree queries per (sequence, head) attend densely to a right-padded
 * per-sequence KV cache of kv_seq_len[b] rows and, under an additive [Q,Q] mask, to
 * the Q new tree tokens; both parts are folded into one softmax.
 *
 * The entry points replace, for a caller that binds native code, the body of the
 * reference's only public function
 *     flash_decoding_attention(q, k_cache, v_cache, current_k, current_v, mask,
 *                              kv_seq_len, block_size, max_seq_len_in_batch, output,
 *                              mid_output, mid_output_lse, sm_scale, kv_group_num)
 * (flash_tree_attn.py:216-376), i.e. its two Triton launches (flash_tree_attn.py:301-334
 * and :340-365), the eager-torch tree tail (:367-371) and the final LSE blend (:373).
 *
 * Conventions: plain pointers and sizes, no C++ or torch types.  All pointers are
 * device pointers unless a name ends in _host.  Strides are in ELEMENTS.  Every tensor
 * must have unit stride in its last (head_dim) dimension.  Every call is asynchronous
 * on the stream it is given, allocates nothing, never synchronises and never throws;
 * the return value is 0 or an FTA_E_* code (fta_strerror gives the text).
 */
#ifndef FTA_H_
#define FTA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 101: FtaExchangeParams.done points at two int32s (scatter form); stage 2 is a programmatic
   dependent launch.  100: first version. */
#define FTA_VERSION 101

/* ---- error codes ------------------------------------------------------------------- */
#define FTA_OK 0
#define FTA_E_BADARG 1      /* a size, stride, dtype or pointer is invalid          */
#define FTA_E_UNSUPPORTED 2 /* a valid request this build has no kernel for         */
#define FTA_E_WORKSPACE 3   /* workspace / mid buffers too small for the plan       */
#define FTA_E_CUDA 4        /* a CUDA runtime or driver call failed                 */
#define FTA_E_TOO_LARGE 5   /* request exceeds the fixed scratch of fta_decode_static */

/* ---- enums ------------------------------------------------------------------------- */
#define FTA_DTYPE_F16 0
#define FTA_DTYPE_BF16 1
#define FTA_DTYPE_F32 2 /* only as out_dtype */

/* how KV rows are divided among thread blocks */
#define FTA_SPLIT_BALANCED 0 /* equal tile ranges per resident block (planner)          */
#define FTA_SPLIT_FIXED 1    /* one partial per split_tokens rows, like the reference's  \
                                one-program-per-block grid (flash_tree_attn.py:295-299)  */

/* which stage-1 kernel family runs */
#define FTA_KERNEL_AUTO 0
#define FTA_KERNEL_MMA 1  /* warp-level mma.sync tiles, cp.async ring                    */
#define FTA_KERNEL_UMMA 2 /* tcgen05 tiles with TMEM accumulators, TMA ring              */

/*
 * One call of the operator.  Shapes (reference docstring, flash_tree_attn.py:236-243,
 * corrected by its index arithmetic :60-94):
 *   q          [B, H,   Q,   D]            query rows of the tree nodes
 *   k_cache    [B, Hkv, ctx, D]            dense right-padded cache (v_cache alike)
 *   current_k  [B, Hkv, Q,   D]            keys of the tree nodes (current_v alike);
 *                                          cur_head_mul selects head kvh*cur_head_mul,
 *                                          so a [B,H,Q,D] tensor is passed with mul = G
 *   mask       fp32, additive, indexed mask[b*m_sb + h*m_sh + i*m_sq + j]; a stride of 0
 *              broadcasts (flash_tree_attn.py:368 adds it to the scaled scores)
 *   kv_seq_len [B] int32 or int64 (flash_tree_attn.py:55)
 * G = H / Hkv consecutive query heads share KV head h / G (flash_tree_attn.py:71).
 */
typedef struct FtaParams {
  /* inputs */
  const void* q;
  int64_t q_sb, q_sh, q_sq;
  const void* k_cache;
  int64_t k_sb, k_sh, k_st;
  const void* v_cache;
  int64_t v_sb, v_sh, v_st;
  const void* cur_k;
  int64_t ck_sb, ck_sh, ck_st;
  const void* cur_v;
  int64_t cv_sb, cv_sh, cv_st;
  const float* mask;
  int64_t m_sb, m_sh, m_sq;
  const void* kv_seq_len;
  int32_t len_is_i64;
  int32_t cur_head_mul;

  /* outputs */
  void* out; /* [B,H,Q,D] merged attention, out_dtype */
  int64_t o_sb, o_sh, o_sq;
  void* out_cache; /* optional: cache-only attention (what the reference leaves in its
                      `output` argument, flash_tree_attn.py:340-365); q dtype; FIXED only */
  int64_t oc_sb, oc_sh, oc_sq;
  float* lse; /* optional [B,H,Q] fp32 natural-log LSE of the merged softmax */
  int64_t l_sb, l_sh;

  /* partial results.  BALANCED: `workspace` of fta_workspace_bytes() bytes.
     FIXED: mid_o [B,H,S,Q,D] / mid_lse [B,H,S,Q] fp32 exactly as the reference lays them
     out (flash_tree_attn.py:276-281), slot s = rows [s*split_tokens,(s+1)*split_tokens);
     tree_o [B,H,Q,D] / tree_lse [B,H,Q] fp32 contiguous hold the tree-token partial. */
  void* workspace;
  int64_t workspace_bytes;
  float* mid_o;
  int64_t mo_sb, mo_sh, mo_ss, mo_sq;
  float* mid_lse;
  int64_t ml_sb, ml_sh, ml_ss;
  int32_t mid_splits; /* S: slots available per (b,h) */
  float* tree_o;
  float* tree_lse;

  /* sizes */
  int32_t B, H, Hkv, Q, D, ctx;
  int32_t dtype;     /* FTA_DTYPE_F16 | FTA_DTYPE_BF16: q, caches, current k/v */
  int32_t out_dtype; /* dtype of `out`: same as dtype, or FTA_DTYPE_F32 */
  float sm_scale;

  /* plan */
  int32_t split_mode;   /* FTA_SPLIT_* */
  int32_t split_tokens; /* FIXED: rows per split, a multiple of 16 */
  int32_t with_tree;    /* 0: cache only (a KV-range shard that does not own the tree) */
  int32_t kernel;       /* FTA_KERNEL_* */
  int32_t grid_override; /* 0 = planner's choice; else resident blocks to launch (tests) */
  int32_t reserved_;

  /* Paged cache (optional; block_table == NULL selects the dense cache above).  k_cache / v_cache
     are then pools of pages [n_pages, Hkv, page_size, D] (k_sb / v_sb = page stride, k_sh, k_st as
     before) and row r of sequence b lives in page block_table[b * bt_sb + r / page_size] at row
     r % page_size.  page_size is a multiple of 64; ctx is the largest kv_seq_len the table can
     hold, i.e. at most bt_sb * page_size.  The reference's docstring announces such a cache
     (flash_tree_attn.py:233) but its kernels index a dense padded one (:72-73); this is the layout
     its README lists as to do. */
  const int32_t* block_table;
  int64_t bt_sb;
  int32_t page_size;
  int32_t n_pages;
} FtaParams;

/*
 * Merge of `n_parts` already-normalised partial attentions (used after the all-gather of
 * KV-range shards): out = sum_s w_s * part_o[s], w_s = softmax_s(part_lse[s]).
 *   part_o   fp32, part_o[s*po_ss + row*D + d], row in [0, rows)
 *   part_lse fp32, part_lse[s*pl_ss + row]
 * It restates flash_tree_attn.py:195-208 for a fixed split count.
 */
typedef struct FtaMergeParams {
  const float* part_o;
  int64_t po_ss;
  const float* part_lse;
  int64_t pl_ss;
  int32_t n_parts;
  int32_t rows;
  int32_t D;
  int32_t out_dtype; /* FTA_DTYPE_* */
  void* out;         /* [rows, D] contiguous */
  float* lse;        /* optional [rows] */
} FtaMergeParams;

/*
 * Exchange + merge of KV-range shard partials between the GPUs of one box, without a library
 * collective: one launch per rank.  No counterpart in the reference (single GPU); the merge is
 * flash_tree_attn.py:195-208 over one partial per rank, in rank order.
 *   part[s]       rank s's packed partial as mapped in THIS process: rows*D floats of O, then
 *                 rows floats of LSE; part[rank] is this rank's own.  Peer entries are device
 *                 pointers of memory mapped from the peer (cuMemMap of an exported handle).
 *   flag_peer[s]  address, as mapped here, of element [rank] of rank s's flag array
 *   flag_local    this rank's flag array [2 * world] (uint32, zero before the first call);
 *                 elements [world, 2 * world) serve the second round of the scatter form
 *   epoch         1, 2, 3, ... (mod 2^32) the same on every rank for the same call
 *   status        device word; bit s is set when the wait for rank s ran out (bit 8 + s: in the
 *                 second round); what was stored by then is not a result.  The word is
 *                 sticky: the kernels only ever set bits, the host clears it after reading
 *   timeout_ns    bound of each wait
 * Two forms.
 *   done == NULL ("gather"): every rank reads every peer's whole partial and writes all rows of
 *     out / lse, which are private to the rank.  One flag round.
 *   done != NULL ("scatter"): rank r merges rows [r * ceil(rows / world), ...) only and stores
 *     them into EVERY rank's result through out_peer[s] / lse_peer[s] (rank s's result buffers as
 *     mapped here; entry [rank] is this rank's own; out and lse are not used); a second flag
 *     round tells the peers that the slice has arrived.  `done` points at two zeroed device
 *     int32s private to the rank (finished blocks; waits lost in the current launch), which the
 *     kernel leaves at zero.  Less NVLink traffic with many ranks: one partial in and half a result out per
 *     GPU instead of (world - 1) partials in.
 * The caller alternates between two partial buffers from call to call (a peer may still read the
 * previous one) and makes the calls in the same order on every rank.  One result buffer per rank
 * is enough: a peer stores into it only after this rank has entered the same call.
 */
#define FTA_MAX_RANKS 8
typedef struct FtaExchangeParams {
  const float* part[FTA_MAX_RANKS];
  uint32_t* flag_peer[FTA_MAX_RANKS];
  void* out_peer[FTA_MAX_RANKS];
  float* lse_peer[FTA_MAX_RANKS];
  const uint32_t* flag_local;
  int32_t* status;
  int32_t* done;
  int64_t timeout_ns;
  int32_t world;
  int32_t rank;
  uint32_t epoch;
  int32_t rows;
  int32_t D;
  int32_t out_dtype; /* FTA_DTYPE_* */
  void* out;         /* [rows, D] contiguous */
  float* lse;        /* optional [rows] */
} FtaExchangeParams;

/* Library / ABI version (FTA_VERSION).  No counterpart in the reference. */
int fta_version(void);

/*
 * Accept/commit, the step after the operator in a speculative-decoding loop: append the accepted
 * tree nodes' keys and values to the cache and grow the lengths.  No counterpart in the reference,
 * which keeps the tree tokens outside the cache (README: "not yet in the cache") and ends there.
 *   cur_k / cur_v   [B, Hkv * cur_head_mul, Q, D] as given to the operator (16-bit elements)
 *   k_cache/v_cache dense [B, Hkv, ctx, D], or pools of pages with block_table as in FtaParams
 *   accept_idx      [B, max_accept] int32, tree-node indices in path order (row stride ai_sb)
 *   accept_len      [B] int32, how many of them count
 *   kv_seq_len      [B] int32/int64, updated in place: += accept_len[b], saturating at ctx
 * Node i of sequence b lands in cache row kv_seq_len[b] + i; rows at or past ctx are dropped.
 */
typedef struct FtaCommitParams {
  const void* cur_k;
  int64_t ck_sb, ck_sh, ck_st;
  const void* cur_v;
  int64_t cv_sb, cv_sh, cv_st;
  void* k_cache;
  int64_t k_sb, k_sh, k_st;
  void* v_cache;
  int64_t v_sb, v_sh, v_st;
  const int32_t* accept_idx;
  int64_t ai_sb;
  const int32_t* accept_len;
  void* kv_seq_len;
  const int32_t* block_table;
  int64_t bt_sb;
  int32_t len_is_i64;
  int32_t cur_head_mul;
  int32_t page_size;
  int32_t n_pages;
  int32_t B, Hkv, Q, D, ctx, max_accept;
} FtaCommitParams;

int fta_commit_accepted(const FtaCommitParams* p, void* stream);

/* Text for an FTA_E_* code.  No counterpart in the reference (it raises AssertionError,
   flash_tree_attn.py:263-291). */
const char* fta_strerror(int code);

/* Last CUDA error text seen by this thread inside the library (for FTA_E_CUDA). */
const char* fta_last_cuda_error(void);

/*
 * Bytes of `workspace` a BALANCED call with these sizes needs on the current device.
 * Replaces the reference's per-call torch.empty of mid_output / mid_output_lse
 * (flash_tree_attn.py:276-281); unlike those it does not grow with B or ctx.
 * Only H, Hkv, Q, D, dtype, kernel and grid_override are read.
 */
int64_t fta_workspace_bytes(const FtaParams* p);

/*
 * The whole operator: stage 1 (split-KV partial attention with the tree-masked tail
 * fused in) and stage 2 (LSE merge), replacing flash_tree_attn.py:301-376.
 * `stream` is a cudaStream_t.  Both kernels are launched with programmatic stream
 * serialization and allow the kernel after them in the stream to be set up early: a
 * kernel the caller launches behind this call WITH that same attribute must, as the
 * attribute's contract says, wait for its grid dependency (cudaGridDependencySynchronize)
 * before it reads `out` / `lse`; an ordinary launch needs nothing.
 */
int fta_decode(const FtaParams* p, void* stream);

/*
 * fta_decode for callers that cannot allocate device memory: a serving runtime that owns the
 * whole device heap and hands none of it out, a plugin loaded into a host process whose
 * allocator it must not touch, code that runs where cudaMalloc is forbidden (inside a stream
 * capture, after the framework has frozen its memory plan).  The caller passes inputs and
 * outputs as for fta_decode; `workspace` and `workspace_bytes` are ignored.  The partial
 * results go to a fixed array inside the library, fta_static_scratch_bytes() bytes (24 MiB)
 * that every GPU loading the library holds until the process exits.  It has no counterpart in
 * the reference, which allocates its partial buffers with torch.empty on every call.
 *
 *  - Only the BALANCED plan is served.  A request whose partial results do not fit the array
 *    (a grid_override far above the device's resident-block count) is refused with
 *    FTA_E_TOO_LARGE; nothing is launched.
 *  - The first call on a device looks up the array's device address (no allocation); make that
 *    first call with the device current and before any stream capture begins.
 *  - All calls on a device share the one array and it keeps whatever the last call left there.
 *    Nothing in it has to start at zero: stage 1 writes every slot stage 2 uses (stage 2 may load
 *    a slot before it knows whether it is needed, and then drops it).  Two calls
 *    whose kernels overlap on the GPU (different streams) race on it; serialise them.
 *  - Neither this function nor anything it calls uses cudaMalloc, cudaFree or an allocating
 *    library routine.
 */
int fta_decode_static(const FtaParams* p, void* stream);

/* Size in bytes of the array fta_decode_static keeps its partial results in.  No counterpart in
   the reference. */
int64_t fta_static_scratch_bytes(void);

/* Stage 1 alone (flash_tree_attn.py:301-334 plus the tail :367-371). */
int fta_stage1(const FtaParams* p, void* stream);

/* Stage 2 alone (flash_tree_attn.py:340-365 plus the blend :373). */
int fta_stage2(const FtaParams* p, void* stream);

/* Merge of gathered shard partials (flash_tree_attn.py:195-208 on a fixed split count). */
int fta_merge_parts(const FtaMergeParams* p, void* stream);

/* Exchange + merge over peer-mapped memory (see FtaExchangeParams). */
int fta_exchange_merge(const FtaExchangeParams* p, void* stream);

/*
 * Host-side evaluation of the BALANCED plan, for tests and tooling: given lengths on
 * the host, report how stage 1 will cut the work.  kv_seq_len_host: [B] int64.
 * segs_out: up to max_segs rows of 8 int64 each
 *   {block, b, unit_in_b, cache_row_begin, cache_row_end, tree_tile_begin, tree_tile_end,
 *    split_index * 65536 + n_splits}.
 * Returns the number of segments (may exceed max_segs; only max_segs are written) or a
 * negative FTA_E_* code.  Replaces the reference's implicit plan "one program per
 * block_size rows" (flash_tree_attn.py:269-274,295-299).
 */
int64_t fta_plan_host(const FtaParams* p, const int64_t* kv_seq_len_host, int64_t* segs_out,
                      int64_t max_segs, int32_t* grid_out, int32_t* per_out);

/*
 * Reads and clears the status word of the tcgen05 stage-1 kernel: 0, or the code of the
 * first bounded barrier wait that gave up (the kernel then returns instead of hanging).
 * Synchronises the device.  No counterpart in the reference.
 */
int fta_umma_status(void);

/* Number of stage-1 thread blocks a call with these sizes launches on the current device. */
int fta_plan_grid(const FtaParams* p);

#ifdef __cplusplus
}
#endif
#endif /* FTA_H_ */
