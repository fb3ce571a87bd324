// C-ABI entry points of libfta.so (declared in include/fta.h): validation, choice of the
// stage-1 kernel family and tile geometry, the resident-grid size the split plan is built
// on, and the launches.  This is the native counterpart of the host body of the reference's
// flash_decoding_attention (flash_tree_attn.py:259-365): its asserts (:263-268,:286-291),
// its implicit plan (:269-274) and its two grids (:295-299,:339).
#include <cstdio>
#include <cstring>
#include <vector>

#include "fta_common.cuh"

cudaError_t fta_launch_stage1_mma_d32(const FtaParams&, const FtaGeom&, cudaStream_t, int, int*);
cudaError_t fta_launch_stage1_mma_d64(const FtaParams&, const FtaGeom&, cudaStream_t, int, int*);
cudaError_t fta_launch_stage1_mma_d128(const FtaParams&, const FtaGeom&, cudaStream_t, int, int*);
cudaError_t fta_launch_stage1_mma_d256(const FtaParams&, const FtaGeom&, cudaStream_t, int, int*);
cudaError_t fta_launch_stage1_umma(const FtaParams&, const FtaGeom&, cudaStream_t, int, int*, int overlap);
int fta_umma_supported(const FtaParams&);
cudaError_t fta_launch_stage2(const FtaParams&, const FtaGeom&, cudaStream_t, int overlap);
cudaError_t fta_launch_commit(const FtaCommitParams&, cudaStream_t);
cudaError_t fta_launch_merge_parts(const FtaMergeParams&, cudaStream_t);
cudaError_t fta_launch_exchange_merge(const FtaExchangeParams&, cudaStream_t);

// Scratch of fta_decode_static: partial results of the BALANCED plan live here instead of in a
// caller-provided workspace.  The array is part of the library image: every GPU that loads the
// library keeps these bytes until the process exits.  In host code the name below is only a
// stand-in for the symbol; the device address is fetched per device with cudaGetSymbolAddress.
#define FTA_STATIC_SCRATCH_BYTES (24u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[FTA_STATIC_SCRATCH_BYTES];

namespace {

void* g_static_scratch_ptr[64];  // device address of g_static_scratch, per device ordinal

thread_local char g_cuda_err[256] = "";

int cuda_fail(cudaError_t e) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return FTA_E_CUDA;
}

bool aligned(const void* ptr, size_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; }
bool mult(int64_t v, int64_t m) { return v % m == 0; }

int validate(const FtaParams* p) {
  if (!p) return FTA_E_BADARG;
  if (p->B <= 0 || p->H <= 0 || p->Hkv <= 0 || p->Q <= 0 || p->ctx < 0) return FTA_E_BADARG;
  if (p->B > FTA_MAX_BATCH) return FTA_E_UNSUPPORTED;
  if (p->H % p->Hkv != 0) return FTA_E_BADARG;
  // head_dim set of the reference (flash_tree_attn.py:263)
  if (p->D != 32 && p->D != 64 && p->D != 128 && p->D != 256) return FTA_E_BADARG;
  if (p->dtype != FTA_DTYPE_F16 && p->dtype != FTA_DTYPE_BF16) return FTA_E_BADARG;
  if (p->out_dtype != p->dtype && p->out_dtype != FTA_DTYPE_F32) return FTA_E_BADARG;
  if (!p->q || !p->kv_seq_len || !p->out) return FTA_E_BADARG;
  if (p->ctx > 0 && (!p->k_cache || !p->v_cache)) return FTA_E_BADARG;
  if (p->with_tree && (!p->cur_k || !p->cur_v || !p->mask || p->cur_head_mul < 1)) return FTA_E_BADARG;
  // 16-byte row chunks are the unit of every copy
  if (!aligned(p->q, 16) || !aligned(p->k_cache, 16) || !aligned(p->v_cache, 16)) return FTA_E_BADARG;
  if (!mult(p->q_sb, 8) || !mult(p->q_sh, 8) || !mult(p->q_sq, 8)) return FTA_E_BADARG;
  if (!mult(p->k_sb, 8) || !mult(p->k_sh, 8) || !mult(p->k_st, 8)) return FTA_E_BADARG;
  if (!mult(p->v_sb, 8) || !mult(p->v_sh, 8) || !mult(p->v_st, 8)) return FTA_E_BADARG;
  if (p->with_tree) {
    if (!aligned(p->cur_k, 16) || !aligned(p->cur_v, 16)) return FTA_E_BADARG;
    if (!mult(p->ck_sb, 8) || !mult(p->ck_sh, 8) || !mult(p->ck_st, 8)) return FTA_E_BADARG;
    if (!mult(p->cv_sb, 8) || !mult(p->cv_sh, 8) || !mult(p->cv_st, 8)) return FTA_E_BADARG;
  }
  if (!aligned(p->out, 16) || !mult(p->o_sb, 4) || !mult(p->o_sh, 4) || !mult(p->o_sq, 4)) return FTA_E_BADARG;
  if (p->block_table) {
    // a 64-row tile never straddles two pages
    if (p->page_size < FTA_TILE || p->page_size % FTA_TILE != 0 || p->n_pages < 1) return FTA_E_BADARG;
    if (p->bt_sb < 0 || (long long)p->bt_sb * p->page_size < p->ctx) return FTA_E_BADARG;
  }
  if (p->split_mode == FTA_SPLIT_BALANCED) {
    if (p->out_cache) return FTA_E_UNSUPPORTED;  // the cache-only result needs FIXED
    if (!p->workspace || !aligned(p->workspace, 16)) return FTA_E_WORKSPACE;
  } else if (p->split_mode == FTA_SPLIT_FIXED) {
    // reference: block_size in {16,32,64,128} (flash_tree_attn.py:268); any multiple of 16 here
    if (p->split_tokens < 16 || p->split_tokens % 16 != 0) return FTA_E_BADARG;
    if (!p->mid_o || !p->mid_lse) return FTA_E_WORKSPACE;
    if (!aligned(p->mid_o, 16) || !mult(p->mo_sb, 4) || !mult(p->mo_sh, 4) || !mult(p->mo_ss, 4) || !mult(p->mo_sq, 4))
      return FTA_E_BADARG;
    // reference: mid buffers must hold kv_max_split_num slots (flash_tree_attn.py:286-288)
    if (p->mid_splits < fta_cdiv(p->ctx, p->split_tokens)) return FTA_E_WORKSPACE;
    if (p->with_tree && (!p->tree_o || !p->tree_lse || !aligned(p->tree_o, 16))) return FTA_E_WORKSPACE;
    if (p->out_cache && (!aligned(p->out_cache, 16) || !mult(p->oc_sb, 4) || !mult(p->oc_sh, 4) || !mult(p->oc_sq, 4)))
      return FTA_E_BADARG;
  } else {
    return FTA_E_BADARG;
  }
  return FTA_OK;
}

// The subset of validate() that the sizing entry points need before make_geom may index its
// tables: sizes, head_dim and dtype (no pointers are read there).
int validate_sizes(const FtaParams* p) {
  if (!p) return FTA_E_BADARG;
  if (p->B <= 0 || p->H <= 0 || p->Hkv <= 0 || p->Q <= 0 || p->ctx < 0) return FTA_E_BADARG;
  if (p->B > FTA_MAX_BATCH) return FTA_E_UNSUPPORTED;
  if (p->H % p->Hkv != 0) return FTA_E_BADARG;
  if (p->D != 32 && p->D != 64 && p->D != 128 && p->D != 256) return FTA_E_BADARG;
  if (p->dtype != FTA_DTYPE_F16 && p->dtype != FTA_DTYPE_BF16) return FTA_E_BADARG;
  return FTA_OK;
}

struct DevInfo {
  int sms = 0;
};
DevInfo g_dev[64];

int dev_info(int* dev, DevInfo** info) {
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return cuda_fail(e);
  DevInfo& d = g_dev[*dev & 63];
  if (d.sms == 0) {
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, *dev);
    if (e != cudaSuccess) return cuda_fail(e);
    d.sms = sms;
  }
  *info = &d;
  return FTA_OK;
}

cudaError_t launch_mma(const FtaParams& p, const FtaGeom& g, cudaStream_t st, int query, int* occ) {
  switch (p.D) {
    case 32: return fta_launch_stage1_mma_d32(p, g, st, query, occ);
    case 64: return fta_launch_stage1_mma_d64(p, g, st, query, occ);
    case 128: return fta_launch_stage1_mma_d128(p, g, st, query, occ);
    case 256: return fta_launch_stage1_mma_d256(p, g, st, query, occ);
  }
  return cudaErrorInvalidValue;
}

// occupancy cache: [device][family][dtype][D index][R index][prefix-table KB]
int g_occ[16][2][2][4][4][34];

int d_index(int D) { return D == 32 ? 0 : D == 64 ? 1 : D == 128 ? 2 : 3; }
int r_index(int R) { return R == 16 ? 0 : R == 32 ? 1 : R == 64 ? 2 : 3; }

int family_of(const FtaParams& p) {
  if (p.kernel == FTA_KERNEL_MMA) return FTA_KERNEL_MMA;
  const bool ok = fta_umma_supported(p) != 0;
  if (p.kernel == FTA_KERNEL_UMMA) return ok ? FTA_KERNEL_UMMA : -1;
  const int M = (p.H / p.Hkv) * p.Q;
  return (ok && M >= 48) ? FTA_KERNEL_UMMA : FTA_KERNEL_MMA;
}

// Tile geometry + resident grid.  no_device: geometry only (grid from grid_override or 1).
int make_geom(const FtaParams& p, FtaGeom& g, bool need_grid) {
  const int fam = family_of(p);
  if (fam < 0) return FTA_E_UNSUPPORTED;
  const int G = p.H / p.Hkv;
  const int M = G * p.Q;
  if (fam == FTA_KERNEL_UMMA) g.R = 128;
  else g.R = (M <= 16) ? 16 : (M <= 32 ? 32 : 64);
  g.qpt = p.Q < g.R ? p.Q : g.R;
  g.hpt = g.R / g.qpt < G ? g.R / g.qpt : G;
  g.n_qt = fta_cdiv(p.Q, g.qpt);
  g.n_gt = fta_cdiv(G, g.hpt);
  g.mtiles = g.n_qt * g.n_gt;
  g.U = p.Hkv * g.mtiles;
  g.n_tree = p.with_tree ? fta_cdiv(p.Q, FTA_TILE) : 0;
  g.min_per = 2;
  g.fixed_max_splits = (p.split_mode == FTA_SPLIT_FIXED && p.split_tokens > 0) ? fta_cdiv(p.ctx, p.split_tokens) : 0;
  g.family = fam;
  g.cs = (fam == FTA_KERNEL_UMMA && g.hpt * g.qpt <= 64) ? 2 : 1;
  // measured cost of ending a unit, in tile times of the family's steady state
  g.pad = (fam == FTA_KERNEL_UMMA && g.cs == 2) ? 8 : 4;
  g.grid = p.grid_override > 0 ? p.grid_override : 1;
  // M tiles of one KV head walk the same tiles in neighbouring blocks (FtaBalanced: lanes)
  g.lanes = (g.mtiles > 1 && g.grid >= g.mtiles) ? g.mtiles : 1;
  if (!need_grid || p.grid_override > 0) return FTA_OK;

  int dev; DevInfo* di;
  int rc = dev_info(&dev, &di);
  if (rc) return rc;
  const int kb = ((p.B + 1) * 4) / 1024;
  int& occ = g_occ[dev & 15][fam == FTA_KERNEL_UMMA][p.dtype][d_index(p.D)][r_index(g.R)][kb < 33 ? kb : 33];
  if (occ == 0) {
    int o = 0;
    cudaError_t e = fam == FTA_KERNEL_UMMA ? fta_launch_stage1_umma(p, g, 0, 1, &o, 0) : launch_mma(p, g, 0, 1, &o);
    if (e != cudaSuccess) return cuda_fail(e);
    if (o < 1) return FTA_E_UNSUPPORTED;
    occ = o;
  }
  g.grid = di->sms * occ;
  g.lanes = (g.mtiles > 1 && g.grid >= g.mtiles) ? g.mtiles : 1;
  return FTA_OK;
}

int64_t ws_bytes(const FtaParams& p, const FtaGeom& g) {
  // partial O + partial LSE for two slots per stage-1 block, then one int4 per stage-1 block
  return (int64_t)2 * g.grid * g.R * (p.D + 1) * 4 + (int64_t)g.grid * 16;
}

// overlap: the two stages are launched with programmatic stream serialization, so that each grid is
// set up while the kernel before it in the stream drains (a whole call); 0 = ordinary launches (a
// stage run alone, e.g. to be timed).
int run_stage1(const FtaParams& p, const FtaGeom& g, cudaStream_t st, int overlap) {
  if (p.split_mode == FTA_SPLIT_BALANCED && p.workspace_bytes < ws_bytes(p, g)) return FTA_E_WORKSPACE;
  cudaError_t e = g.family == FTA_KERNEL_UMMA ? fta_launch_stage1_umma(p, g, st, 0, nullptr, overlap)
                                            : launch_mma(p, g, st, 0, nullptr);
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

}  // namespace

extern "C" {

int fta_version(void) { return FTA_VERSION; }

const char* fta_strerror(int code) {
  switch (code) {
    case FTA_OK: return "ok";
    case FTA_E_BADARG: return "invalid argument (size, stride, alignment, dtype or null pointer)";
    case FTA_E_UNSUPPORTED: return "request not supported by this build";
    case FTA_E_WORKSPACE: return "workspace or mid_output buffers missing or too small";
    case FTA_E_CUDA: return "CUDA call failed (see fta_last_cuda_error)";
    case FTA_E_TOO_LARGE: return "request exceeds the static scratch of the no-allocation entry point";
  }
  return "unknown error";
}

const char* fta_last_cuda_error(void) { return g_cuda_err; }

int64_t fta_workspace_bytes(const FtaParams* p) {
  if (int rc = validate_sizes(p)) return -rc;
  FtaParams q = *p;
  q.split_mode = FTA_SPLIT_BALANCED;
  FtaGeom g;
  int rc = make_geom(q, g, true);
  if (rc) return -rc;
  return ws_bytes(q, g);
}

int fta_plan_grid(const FtaParams* p) {
  if (int rc = validate_sizes(p)) return -rc;
  FtaGeom g;
  int rc = make_geom(*p, g, true);
  return rc ? -rc : g.grid;
}

int fta_stage1(const FtaParams* p, void* stream) {
  int rc = validate(p);
  if (rc) return rc;
  FtaGeom g;
  rc = make_geom(*p, g, true);
  if (rc) return rc;
  return run_stage1(*p, g, (cudaStream_t)stream, 0);
}

int fta_stage2(const FtaParams* p, void* stream) {
  int rc = validate(p);
  if (rc) return rc;
  FtaGeom g;
  rc = make_geom(*p, g, true);
  if (rc) return rc;
  cudaError_t e = fta_launch_stage2(*p, g, (cudaStream_t)stream, 0);
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

int fta_decode(const FtaParams* p, void* stream) {
  int rc = validate(p);
  if (rc) return rc;
  FtaGeom g;
  rc = make_geom(*p, g, true);
  if (rc) return rc;
  rc = run_stage1(*p, g, (cudaStream_t)stream, 1);
  if (rc) return rc;
  cudaError_t e = fta_launch_stage2(*p, g, (cudaStream_t)stream, 1);
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

int64_t fta_static_scratch_bytes(void) { return (int64_t)FTA_STATIC_SCRATCH_BYTES; }

int fta_decode_static(const FtaParams* p, void* stream) {
  if (!p) return FTA_E_BADARG;
  if (p->split_mode != FTA_SPLIT_BALANCED) return FTA_E_UNSUPPORTED;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return FTA_E_UNSUPPORTED;
  if (g_static_scratch_ptr[dev] == nullptr) {
    // first call on this device (made with the device current): resolve the symbol's address
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e);
    if (ptr == nullptr) return FTA_E_CUDA;
    g_static_scratch_ptr[dev] = ptr;
  }
  FtaParams q = *p;
  q.workspace = g_static_scratch_ptr[dev];
  q.workspace_bytes = (int64_t)FTA_STATIC_SCRATCH_BYTES;
  int rc = validate(&q);
  if (rc) return rc;
  FtaGeom g;
  rc = make_geom(q, g, true);
  if (rc) return rc;
  if (ws_bytes(q, g) > (int64_t)FTA_STATIC_SCRATCH_BYTES) return FTA_E_TOO_LARGE;
  rc = run_stage1(q, g, (cudaStream_t)stream, 1);
  if (rc) return rc;
  e = fta_launch_stage2(q, g, (cudaStream_t)stream, 1);
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

int fta_merge_parts(const FtaMergeParams* p, void* stream) {
  if (!p || !p->part_o || !p->part_lse || !p->out) return FTA_E_BADARG;
  if (p->n_parts < 1 || p->rows < 0 || p->D < 4 || p->D % 4 != 0) return FTA_E_BADARG;
  if (!aligned(p->part_o, 16) || !aligned(p->out, 16) || !mult(p->po_ss, 4)) return FTA_E_BADARG;
  if (p->out_dtype < FTA_DTYPE_F16 || p->out_dtype > FTA_DTYPE_F32) return FTA_E_BADARG;
  if (p->rows == 0) return FTA_OK;
  cudaError_t e = fta_launch_merge_parts(*p, (cudaStream_t)stream);
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

int fta_exchange_merge(const FtaExchangeParams* p, void* stream) {
  if (!p || !p->flag_local || !p->status) return FTA_E_BADARG;
  if (p->world < 1 || p->world > FTA_MAX_RANKS || p->rank < 0 || p->rank >= p->world) return FTA_E_BADARG;
  if (p->rows < 0 || p->D < 4 || p->D % 4 != 0 || p->timeout_ns <= 0) return FTA_E_BADARG;
  if (p->out_dtype < FTA_DTYPE_F16 || p->out_dtype > FTA_DTYPE_F32) return FTA_E_BADARG;
  const bool scatter = p->done != nullptr;
  if (!scatter && (!p->out || !aligned(p->out, 16))) return FTA_E_BADARG;
  for (int s = 0; s < p->world; ++s) {
    if (!p->part[s] || !aligned(p->part[s], 16)) return FTA_E_BADARG;
    if (s != p->rank && (!p->flag_peer[s] || !aligned(p->flag_peer[s], 4))) return FTA_E_BADARG;
    if (scatter && (!p->out_peer[s] || !aligned(p->out_peer[s], 16) || !p->lse_peer[s])) return FTA_E_BADARG;
  }
  if (p->rows == 0) return FTA_OK;
  cudaError_t e = fta_launch_exchange_merge(*p, (cudaStream_t)stream);
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

int fta_commit_accepted(const FtaCommitParams* p, void* stream) {
  if (!p || !p->cur_k || !p->cur_v || !p->k_cache || !p->v_cache || !p->accept_idx || !p->accept_len || !p->kv_seq_len)
    return FTA_E_BADARG;
  if (p->B <= 0 || p->Hkv <= 0 || p->Q <= 0 || p->ctx <= 0 || p->max_accept < 0 || p->cur_head_mul < 1) return FTA_E_BADARG;
  if (p->D <= 0 || p->D % 8 != 0) return FTA_E_BADARG;
  if (!aligned(p->cur_k, 16) || !aligned(p->cur_v, 16) || !aligned(p->k_cache, 16) || !aligned(p->v_cache, 16)) return FTA_E_BADARG;
  if (!mult(p->ck_sb, 8) || !mult(p->ck_sh, 8) || !mult(p->ck_st, 8) || !mult(p->cv_sb, 8) || !mult(p->cv_sh, 8) || !mult(p->cv_st, 8))
    return FTA_E_BADARG;
  if (!mult(p->k_sb, 8) || !mult(p->k_sh, 8) || !mult(p->k_st, 8) || !mult(p->v_sb, 8) || !mult(p->v_sh, 8) || !mult(p->v_st, 8))
    return FTA_E_BADARG;
  if (p->block_table && (p->page_size < 1 || p->n_pages < 1 || (long long)p->bt_sb * p->page_size < p->ctx)) return FTA_E_BADARG;
  if (p->max_accept == 0) return FTA_OK;
  cudaError_t e = fta_launch_commit(*p, (cudaStream_t)stream);
  return e == cudaSuccess ? FTA_OK : cuda_fail(e);
}

int64_t fta_plan_host(const FtaParams* p, const int64_t* lens, int64_t* segs_out, int64_t max_segs,
                      int32_t* grid_out, int32_t* per_out) {
  if (!lens) return -FTA_E_BADARG;
  if (int rc = validate_sizes(p)) return -rc;
  FtaParams q = *p;
  q.split_mode = FTA_SPLIT_BALANCED;
  FtaGeom g;
  int rc = make_geom(q, g, true);
  if (rc) return -rc;
  std::vector<int> pre(q.B + 1, 0);
  for (int b = 0; b < q.B; ++b) {
    const int L = fta_load_len(lens, 1, b, q.ctx);
    pre[b + 1] = pre[b] + fta_unit_tiles(L, g.n_tree, g.pad);
  }
  FtaBalanced plan;
  plan.init(pre.data(), q.B, g, g.grid);
  if (grid_out) *grid_out = g.grid;
  if (per_out) *per_out = plan.per;
  int64_t n = 0;
  for (int c = 0; c < g.grid; ++c) {
    long long lin = 0, end = 0;
    if (!plan.range(c, g.grid, lin, end)) continue;
    while (lin < end) {
      FtaSeg s;
      lin = plan.segment_at(c, lin, s);
      if (fta_seg_empty(s)) continue;
      const int L = fta_load_len(lens, 1, s.b, q.ctx);
      if (s.c1 > L) s.c1 = L;
      if (segs_out && n < max_segs) {
        int64_t* o = segs_out + n * 8;
        o[0] = c; o[1] = s.b; o[2] = s.j; o[3] = s.c0; o[4] = s.c1; o[5] = s.tt0; o[6] = s.tt1;
        o[7] = (int64_t)s.split * 65536 + s.nsplit;
      }
      ++n;
    }
  }
  return n;
}

}  // extern "C"
