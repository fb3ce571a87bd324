// Stage 1, warp-MMA family: split-KV tree attention on mma.sync.m16n8k16 tiles fed by a
// cp.async ring.  It serves every shape (any Q, G, D in {32,64,128,256}); it is the path
// of choice when M = G*Q is small, where the KV stream is the only cost.
//
// It replaces the reference's _flash_decoding_fwd_kernel (flash_tree_attn.py:14-144) and,
// fused into the same block, the eager tree tail (flash_tree_attn.py:367-371).
// Differences by design: all G*Q rows that share a KV head form one tile (the reference
// re-reads the KV block once per query head, :51,71-73); a block walks many 64-row tiles
// with an online softmax instead of one block_size slice (:49-57); KV rows past
// kv_seq_len[b] are never read (zero-filled), so the padding may hold anything.
#pragma once
#include "fta_common.cuh"

namespace fta_mma {

constexpr int kThreads = 128;

template <int D> struct StageCount { static constexpr int v = D <= 32 ? 6 : (D <= 64 ? 5 : (D <= 128 ? 3 : 2)); };

template <int D, int WM, int WN>
struct Cfg {
  static constexpr int R = 16 * WM;
  static constexpr int TN = FTA_TILE / WN;  // KV rows of a tile handled by one warp
  static constexpr int ROWB = D * 2;
  static constexpr int CH = D / 8;  // 16-byte chunks per row
  static constexpr int STAGES = StageCount<D>::v;
  static constexpr int Q_BYTES = R * ROWB;
  static constexpr int STAGE_BYTES = 2 * FTA_TILE * ROWB;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int EPITCH = D + 8;  // floats
  static constexpr int EPI_BYTES = WN * R * EPITCH * 4 + 2 * WN * R * 4;
  static constexpr int BODY_BYTES = RING_BYTES > EPI_BYTES ? RING_BYTES : EPI_BYTES;
  static constexpr int FIXED_BYTES = Q_BYTES + BODY_BYTES;
  static constexpr bool Q_IN_REGS = D <= 128;
};

template <int CH> __device__ __forceinline__ int swz(int row, int chunk) {
  if (CH >= 8) return chunk ^ (row & 7);
  return chunk ^ ((row >> 1) & (CH - 1));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Copy FTA_TILE rows of D elements (row i at g + i*stride) into a swizzled tile; rows at or
// past `valid` are zero-filled without touching memory.  Each thread owns one 16-byte column
// chunk and walks down the rows, so its swizzled shared-memory offset is a constant plus a
// multiple of the pass pitch.
template <typename T, int D>
__device__ __forceinline__ void load_rows(uint32_t sdst, const T* g, long long stride, int valid) {
  constexpr int CH = D / 8;
  constexpr int RPP = kThreads / CH;  // rows per pass
  const int ch = threadIdx.x % CH, r0 = threadIdx.x / CH;
  const T* src = g + (long long)r0 * stride + ch * 8;
  const long long step = (long long)RPP * stride;
  const uint32_t d0 = sdst + r0 * (D * 2);
  const uint32_t sw_const = (uint32_t)swz<CH>(r0, ch) << 4;
#pragma unroll
  for (int k = 0; k < FTA_TILE / RPP; ++k) {
    const int row = r0 + k * RPP;
    const bool ok = row < valid;
    const uint32_t sw = (RPP % 8 == 0 || CH < 8) ? sw_const : ((uint32_t)swz<CH>(row, ch) << 4);
    cp_async16(d0 + k * RPP * (D * 2) + sw, ok ? src : g, ok ? 16 : 0);
    src += step;
  }
}

template <typename T, int D, int WM, int WN>
__global__ void __launch_bounds__(kThreads, (Cfg<D, WM, WN>::FIXED_BYTES <= 112 * 1024) ? 2 : 1)
stage1_kernel(const FtaParams p, const FtaGeom g) {
  using C = Cfg<D, WM, WN>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sBody = smem + C::Q_BYTES;
  int* pre = reinterpret_cast<int*>(smem + C::FIXED_BYTES);
  const uint32_t sQ_a = (uint32_t)__cvta_generic_to_shared(sQ);
  const uint32_t sBody_a = (uint32_t)__cvta_generic_to_shared(sBody);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / WN, wn = warp % WN;
  const int gq = lane >> 2, tq = lane & 3;  // mma fragment coordinates
  const int G = p.H / p.Hkv;
  const float scale2 = p.sm_scale * FTA_LOG2E;
  const T* Qp = (const T*)p.q;
  const T* Kp = (const T*)p.k_cache;
  const T* Vp = (const T*)p.v_cache;
  const T* CKp = (const T*)p.cur_k;
  const T* CVp = (const T*)p.cur_v;

  // stage 2 is launched with programmatic stream serialization: let its grid be set up now; its
  // blocks wait for this whole grid to finish before they read anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  FtaBalanced plan;
  long long lin = 0, lin_end = 0, item = 0, n_items = 0;
  if (p.split_mode == FTA_SPLIT_BALANCED) {
    fta_build_prefix(p, g.n_tree, g.pad, pre);
    __syncthreads();
    plan.init(pre, p.B, g, gridDim.x);
    if (!plan.range(blockIdx.x, gridDim.x, lin, lin_end)) lin = lin_end = 0;
    if (tid == 0) fta_cut_desc(p, g)[blockIdx.x] = make_int4(0, 0, 0, 0);  // rewritten below if a cut unit opens this block
  } else {
    item = blockIdx.x;
    n_items = (long long)p.B * g.U * (g.fixed_max_splits + 1);
  }

  for (;;) {
    // ---- next piece of work ------------------------------------------------------------
    FtaSeg seg;
    int Lb;
    if (p.split_mode == FTA_SPLIT_BALANCED) {
      if (lin >= lin_end) break;
      lin = plan.segment_at(blockIdx.x, lin, seg);
      if (fta_seg_empty(seg)) continue;  // only the virtual tail of a unit
      Lb = fta_load_len(p.kv_seq_len, p.len_is_i64, seg.b, p.ctx);
      if (seg.c1 > Lb) seg.c1 = Lb;
    } else {
      if (item >= n_items) break;
      const int per_unit = g.fixed_max_splits + 1;
      const long long per_b = (long long)g.U * per_unit;
      seg.b = (int)(item / per_b);
      const long long r = item - (long long)seg.b * per_b;
      seg.j = (int)(r / per_unit);
      seg.split = (int)(r - (long long)seg.j * per_unit);
      item += gridDim.x;
      Lb = fta_load_len(p.kv_seq_len, p.len_is_i64, seg.b, p.ctx);
      seg.nsplit = 0; seg.slot = 0;
      if (seg.split == g.fixed_max_splits) {  // tree piece
        if (g.n_tree == 0) continue;
        seg.c0 = seg.c1 = 0; seg.tt0 = 0; seg.tt1 = g.n_tree;
      } else {
        seg.c0 = seg.split * p.split_tokens;
        if (seg.c0 >= Lb) continue;
        seg.c1 = seg.c0 + p.split_tokens < Lb ? seg.c0 + p.split_tokens : Lb;
        seg.tt0 = seg.tt1 = 0;
      }
    }
    const int n_ct = seg.c1 > seg.c0 ? fta_cdiv(seg.c1 - seg.c0, FTA_TILE) : 0;
    const int n_tiles = n_ct + (seg.tt1 - seg.tt0);
    const FtaUnit unit = fta_unit(g, seg.j);

    // per-thread rows: r0 = 16*wm + gq, r1 = r0 + 8
    int row_h[2], row_q[2];
    bool row_ok[2];
    const float* mrow[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      row_ok[e] = fta_row(p, g, unit, 16 * wm + gq + 8 * e, row_h[e], row_q[e]);
      mrow[e] = row_ok[e] ? p.mask + seg.b * p.m_sb + row_h[e] * p.m_sh + row_q[e] * p.m_sq : nullptr;
    }

    const T* kbase = Kp + unit.kvh * p.k_sh;  // + the tile's batch / page and row
    const T* vbase = Vp + unit.kvh * p.v_sh;
    const T* ckbase = CKp + seg.b * p.ck_sb + (long long)unit.kvh * p.cur_head_mul * p.ck_sh;
    const T* cvbase = CVp + seg.b * p.cv_sb + (long long)unit.kvh * p.cur_head_mul * p.cv_sh;

    // where cache tile i starts (paged cache: a block-table read); asked one tile ahead of its use,
    // so that no copy is issued behind a table read
    auto tile_at = [&](int i) {
      FtaTileAt at = {0, 0};
      if (i < n_ct) at = fta_tile_at(p, seg.b, seg.c0 + i * FTA_TILE);
      return at;
    };
    auto issue_tile = [&](int i, const FtaTileAt& at) {
      if (i < n_tiles) {
        const uint32_t sK = sBody_a + (i % C::STAGES) * C::STAGE_BYTES;
        const uint32_t sV = sK + FTA_TILE * C::ROWB;
        if (i < n_ct) {
          const int row0 = seg.c0 + i * FTA_TILE;
          const int valid = seg.c1 - row0 < FTA_TILE ? seg.c1 - row0 : FTA_TILE;
          load_rows<T, D>(sK, kbase + at.batch * p.k_sb + (long long)at.row * p.k_st, p.k_st, valid);
          load_rows<T, D>(sV, vbase + at.batch * p.v_sb + (long long)at.row * p.v_st, p.v_st, valid);
        } else {
          const int row0 = (seg.tt0 + i - n_ct) * FTA_TILE;
          const int valid = p.Q - row0 < FTA_TILE ? p.Q - row0 : FTA_TILE;
          load_rows<T, D>(sK, ckbase + (long long)row0 * p.ck_st, p.ck_st, valid);
          load_rows<T, D>(sV, cvbase + (long long)row0 * p.cv_st, p.cv_st, valid);
        }
      }
      cp_async_commit();
    };

    // ---- Q tile + pipeline prologue ------------------------------------------------------
    for (int i = tid; i < C::R * C::CH; i += kThreads) {
      const int row = i / C::CH, ch = i - row * C::CH;
      int h, qi;
      const bool ok = fta_row(p, g, unit, row, h, qi);
      const T* src = ok ? Qp + seg.b * p.q_sb + h * p.q_sh + qi * p.q_sq + ch * 8 : Qp;
      cp_async16(sQ_a + row * C::ROWB + (swz<C::CH>(row, ch) << 4), src, ok ? 16 : 0);
    }
    {
      FtaTileAt first[C::STAGES - 1];
#pragma unroll
      for (int i = 0; i < C::STAGES - 1; ++i) first[i] = tile_at(i);  // the reads go out together
#pragma unroll
      for (int i = 0; i < C::STAGES - 1; ++i) issue_tile(i, first[i]);
    }
    FtaTileAt at_next = tile_at(C::STAGES - 1);

    uint32_t qf[C::Q_IN_REGS ? D / 16 : 1][4];
    float acc_o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { acc_o[i][0] = acc_o[i][1] = acc_o[i][2] = acc_o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // ---- main loop over KV tiles -----------------------------------------------------------
    for (int i = 0; i < n_tiles; ++i) {
      cp_async_wait<C::STAGES - 2>();
      __syncthreads();
      issue_tile(i + C::STAGES - 1, at_next);
      at_next = tile_at(i + C::STAGES);

      if (C::Q_IN_REGS && i == 0) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const int row = 16 * wm + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int ch = ks * 2 + (lane >> 4);
          ldsm_x4(sQ_a + row * C::ROWB + (swz<C::CH>(row, ch) << 4), qf[C::Q_IN_REGS ? ks : 0][0],
                  qf[C::Q_IN_REGS ? ks : 0][1], qf[C::Q_IN_REGS ? ks : 0][2], qf[C::Q_IN_REGS ? ks : 0][3]);
        }
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
      if (wn * C::TN >= valid) continue;  // this warp's KV rows are all padding

      const uint32_t sK = sBody_a + (i % C::STAGES) * C::STAGE_BYTES;
      const uint32_t sV = sK + FTA_TILE * C::ROWB;

      // S = Q K^T over this warp's TN KV rows
      float acc_s[C::TN / 8][4];
#pragma unroll
      for (int n = 0; n < C::TN / 8; ++n) { acc_s[n][0] = acc_s[n][1] = acc_s[n][2] = acc_s[n][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a[4];
        if (C::Q_IN_REGS) {
          a[0] = qf[C::Q_IN_REGS ? ks : 0][0]; a[1] = qf[C::Q_IN_REGS ? ks : 0][1];
          a[2] = qf[C::Q_IN_REGS ? ks : 0][2]; a[3] = qf[C::Q_IN_REGS ? ks : 0][3];
        } else {
          const int row = 16 * wm + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int ch = ks * 2 + (lane >> 4);
          ldsm_x4(sQ_a + row * C::ROWB + (swz<C::CH>(row, ch) << 4), a[0], a[1], a[2], a[3]);
        }
#pragma unroll
        for (int n = 0; n < C::TN / 8; n += 2) {
          const int row = wn * C::TN + n * 8 + (lane >> 4) * 8 + (lane & 7);
          const int ch = ks * 2 + ((lane >> 3) & 1);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(sK + row * C::ROWB + (swz<C::CH>(row, ch) << 4), b0, b1, b2, b3);
          mma16816<T>(acc_s[n], a, b0, b1);
          mma16816<T>(acc_s[n + 1], a, b2, b3);
        }
      }

      // scale, mask, online softmax (rows gq and gq+8 of this warp's 16)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < C::TN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = wn * C::TN + n * 8 + 2 * tq + (e & 1);
          const int r = e >> 1;
          float s = acc_s[n][e] * scale2;
          if (is_tree && col < valid && mrow[r] != nullptr) s += __ldg(mrow[r] + col0 + col) * FTA_LOG2E;
          if (col >= valid) s = -INFINITY;
          acc_s[n][e] = s;
          mx[r] = fmaxf(mx[r], s);
        }
      }
      float alpha[2], msafe[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mnew = fmaxf(m_run[r], mx[r]);
        msafe[r] = mnew == -INFINITY ? 0.f : mnew;
        alpha[r] = fta_exp2(m_run[r] - msafe[r]);
        m_run[r] = mnew;
      }
      float psum[2] = {0.f, 0.f};
#pragma unroll
      for (int n = 0; n < C::TN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = fta_exp2(acc_s[n][e] - msafe[e >> 1]);
          acc_s[n][e] = pv;
          psum[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + psum[r];
#pragma unroll
      for (int dn = 0; dn < D / 8; ++dn) {
        acc_o[dn][0] *= alpha[0]; acc_o[dn][1] *= alpha[0];
        acc_o[dn][2] *= alpha[1]; acc_o[dn][3] *= alpha[1];
      }

      // O += P V
#pragma unroll
      for (int kj = 0; kj < C::TN / 16; ++kj) {
        uint32_t a[4];
        a[0] = FtaType<T>::pack(acc_s[2 * kj][0], acc_s[2 * kj][1]);
        a[1] = FtaType<T>::pack(acc_s[2 * kj][2], acc_s[2 * kj][3]);
        a[2] = FtaType<T>::pack(acc_s[2 * kj + 1][0], acc_s[2 * kj + 1][1]);
        a[3] = FtaType<T>::pack(acc_s[2 * kj + 1][2], acc_s[2 * kj + 1][3]);
#pragma unroll
        for (int dn = 0; dn < D / 8; dn += 2) {
          const int row = wn * C::TN + kj * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int ch = dn + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(sV + row * C::ROWB + (swz<C::CH>(row, ch) << 4), b0, b1, b2, b3);
          mma16816<T>(acc_o[dn], a, b0, b1);
          mma16816<T>(acc_o[dn + 1], a, b2, b3);
        }
      }
    }

    // ---- epilogue: combine the WN warps of a row group, normalise, store ---------------------
    cp_async_wait<0>();
    __syncthreads();
    float* eO = reinterpret_cast<float*>(sBody);
    float* eM = eO + WN * C::R * C::EPITCH;
    float* eL = eM + WN * C::R;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    {
      const int r0 = 16 * wm + gq;
      float* o0 = eO + (wn * C::R + r0) * C::EPITCH;
      float* o1 = o0 + 8 * C::EPITCH;
#pragma unroll
      for (int dn = 0; dn < D / 8; ++dn) {
        *reinterpret_cast<float2*>(o0 + dn * 8 + 2 * tq) = make_float2(acc_o[dn][0], acc_o[dn][1]);
        *reinterpret_cast<float2*>(o1 + dn * 8 + 2 * tq) = make_float2(acc_o[dn][2], acc_o[dn][3]);
      }
      if (tq == 0) {
        eM[wn * C::R + r0] = m_run[0]; eM[wn * C::R + r0 + 8] = m_run[1];
        eL[wn * C::R + r0] = l_run[0]; eL[wn * C::R + r0 + 8] = l_run[1];
      }
    }
    __syncthreads();

    const bool final_direct = p.split_mode == FTA_SPLIT_BALANCED && seg.nsplit == 1;
    const bool tree_piece = p.split_mode == FTA_SPLIT_FIXED && seg.split == g.fixed_max_splits;
    float* ws_o = reinterpret_cast<float*>(p.workspace);
    float* ws_l = ws_o + (long long)2 * g.grid * g.R * D;
    if (p.split_mode == FTA_SPLIT_BALANCED && seg.split == 1 && tid == 0)
      fta_cut_desc(p, g)[blockIdx.x] = make_int4(seg.b, seg.j, seg.nsplit, seg.p0slot);  // for stage 2
    for (int i = tid; i < C::R * (D / 4); i += kThreads) {
      const int row = i / (D / 4), c4 = (i - row * (D / 4)) * 4;
      int h, qi;
      if (!fta_row(p, g, unit, row, h, qi)) continue;
      float mstar = -INFINITY;
#pragma unroll
      for (int w = 0; w < WN; ++w) mstar = fmaxf(mstar, eM[w * C::R + row]);
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
      float l = 0.f;
      if (mstar != -INFINITY) {
#pragma unroll
        for (int w = 0; w < WN; ++w) {
          const float wgt = fta_exp2(eM[w * C::R + row] - mstar);
          const float4 v = *reinterpret_cast<const float4*>(eO + (w * C::R + row) * C::EPITCH + c4);
          o.x += wgt * v.x; o.y += wgt * v.y; o.z += wgt * v.z; o.w += wgt * v.w;
          l += wgt * eL[w * C::R + row];
        }
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      o.x *= inv; o.y *= inv; o.z *= inv; o.w *= inv;
      const float lse = l > 0.f ? (mstar + fta_log2(l)) * FTA_LN2 : -INFINITY;
      if (final_direct) {
        fta_store4(p.out, p.out_dtype, seg.b * p.o_sb + h * p.o_sh + qi * p.o_sq + c4, o);
        if (c4 == 0 && p.lse) p.lse[seg.b * p.l_sb + h * p.l_sh + qi] = lse;
      } else if (p.split_mode == FTA_SPLIT_BALANCED) {
        *reinterpret_cast<float4*>(ws_o + ((long long)seg.slot * g.R + row) * D + c4) = o;
        if (c4 == 0) ws_l[(long long)seg.slot * g.R + row] = lse;
      } else if (tree_piece) {
        const long long ro = ((long long)seg.b * p.H + h) * p.Q + qi;
        *reinterpret_cast<float4*>(p.tree_o + ro * D + c4) = o;
        if (c4 == 0) p.tree_lse[ro] = lse;
      } else {
        *reinterpret_cast<float4*>(p.mid_o + seg.b * p.mo_sb + h * p.mo_sh + seg.split * p.mo_ss + qi * p.mo_sq + c4) = o;
        if (c4 == 0) p.mid_lse[seg.b * p.ml_sb + h * p.ml_sh + seg.split * p.ml_ss + qi] = lse;
      }
    }
    __syncthreads();
  }
}

}  // namespace fta_mma
