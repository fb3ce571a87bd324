// Accept/commit: the step right after the tree-attention verification.  The verifier has picked,
// for every sequence, the tree nodes that are accepted (a root-to-leaf path, in order); their keys
// and values, which the operator deliberately keeps outside the cache (`current_k`, `current_v`),
// are appended to the cache at rows kv_seq_len[b], kv_seq_len[b] + 1, ... and the lengths grow by
// the number accepted.  The reference stops before this step (its README describes the tree tokens
// as "not yet in the cache" and lists cache management as to do); nothing of it is restated here.
//
// Pure data movement: 2 * 2 * D bytes read and written per accepted token and KV head, in 16-byte
// chunks.  Rows that would land at or past ctx are dropped and the length saturates at ctx.
#include "fta_common.cuh"

namespace {

constexpr int kThreads = 256;

// grid = (B, Hkv).  Lengths are read here and bumped by a second kernel: a block that started
// late must not see a length another block of the same sequence has already moved.
__global__ void __launch_bounds__(kThreads) commit_rows_kernel(const FtaCommitParams p) {
  const int b = blockIdx.x, kvh = blockIdx.y;
  int n = p.accept_len[b];
  if (n > p.max_accept) n = p.max_accept;
  if (n <= 0) return;
  const int L = fta_load_len(p.kv_seq_len, p.len_is_i64, b, p.ctx);
  const int chunks = p.D / 8;  // 16-byte chunks of a row (16-bit elements)
  const uint4* ck = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.cur_k) + b * p.ck_sb +
                                                   (long long)kvh * p.cur_head_mul * p.ck_sh);
  const uint4* cv = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.cur_v) + b * p.cv_sb +
                                                   (long long)kvh * p.cur_head_mul * p.cv_sh);
  for (int idx = threadIdx.x; idx < n * chunks; idx += kThreads) {
    const int i = idx / chunks, c = idx - i * chunks;
    const int row = L + i;
    if (row >= p.ctx) continue;
    const int node = p.accept_idx[b * p.ai_sb + i];
    if (node < 0 || node >= p.Q) continue;  // an invalid index copies nothing
    int batch = b, r = row;
    if (p.block_table != nullptr) {
      const int slot = row / p.page_size;
      batch = p.block_table[(long long)b * p.bt_sb + slot];
      r = row - slot * p.page_size;
    }
    uint16_t* kd = reinterpret_cast<uint16_t*>(p.k_cache) + batch * p.k_sb + kvh * p.k_sh + (long long)r * p.k_st;
    uint16_t* vd = reinterpret_cast<uint16_t*>(p.v_cache) + batch * p.v_sb + kvh * p.v_sh + (long long)r * p.v_st;
    reinterpret_cast<uint4*>(kd)[c] = ck[(node * p.ck_st) / 8 + c];
    reinterpret_cast<uint4*>(vd)[c] = cv[(node * p.cv_st) / 8 + c];
  }
}

__global__ void bump_lengths_kernel(const FtaCommitParams p) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= p.B) return;
  int n = p.accept_len[b];
  if (n > p.max_accept) n = p.max_accept;
  if (n <= 0) return;
  long long L = fta_load_len(p.kv_seq_len, p.len_is_i64, b, p.ctx) + (long long)n;
  if (L > p.ctx) L = p.ctx;
  if (p.len_is_i64) reinterpret_cast<long long*>(p.kv_seq_len)[b] = L;
  else reinterpret_cast<int*>(p.kv_seq_len)[b] = (int)L;
}

}  // namespace

cudaError_t fta_launch_commit(const FtaCommitParams& p, cudaStream_t st) {
  commit_rows_kernel<<<dim3(p.B, p.Hkv), kThreads, 0, st>>>(p);
  bump_lengths_kernel<<<(p.B + 127) / 128, 128, 0, st>>>(p);
  return cudaGetLastError();
}
