// tcgen05 / TMA version of the chunk-parallel output kernels (bf16 / fp16, K in {64,128}, V % 64 == 0):
//   fwd_o    : o  = scale * [(q h) * e^{b_i} + tril(q k^T * e^{b_i-b_j}) v]      (fla/ops/common/chunk_o.py:23-101)
//   bwd_dv   : dv = (k dh) * e^{b_L-b_j} + triu(k q^T * e^{b_i-b_j}) * scale do  (fla/ops/common/chunk_o.py:289-364)
//   dv_local : second term of bwd_dv only                                         (fla/ops/common/chunk_o.py:379-441)
//
// Persistent kernel, one CTA per SM, work item = (chunk, head, 128-wide V tile).  Nineteen warps:
//   warp 16 : TMA producer  - streams the item's tiles (x1, x2, y, state) into a ring of stages; a stage has two halves
//                             with barriers of their own: x1 | x2 | state is dead as soon as the first two products have
//                             run, so it is refilled for a later item while the epilogue still works on this one and only
//                             y waits for the item's last product
//   warp 17 : MMA issuer    - S = x1 x2^T and O = x1 state into TMEM, later O = P y
//   warps 0-7 / 8-15: two epilogue groups working on even / odd items (ping-pong); inside a group
//                     warp = (TMEM lane quadrant = 16 token rows, column half)
//                           - S -> mask / decay -> P (bf16, swizzled shared memory); O -> gate -> out
//   warp 18 : scalars       - gates and row count of the coming items into a ring of four shared-memory slots, so that no
//                             epilogue warp ever waits for a global load; its first lane also issues the tile stores of
//                             the finished output tiles (three items behind the gates) and frees the groups' output
//                             buffers, so that no epilogue warp issues a store or waits for one either
// The epilogue warps meet each other only through the mbarriers of the phases (one arrival per warp), never through a
// barrier of the group.
// The epilogue arithmetic (one exponential per score element, packing, swizzled stores) is what
// bounds the kernel, hence 16 epilogue warps for one MMA-issuing thread.
// TMEM holds two stages of [S: 64 columns | O: 128 columns] (M = 64 rows = lanes 0-15 of each warp's
// quadrant), one per epilogue group, so the tensor core and the other group work on item i+1 while
// one group finishes item i.  The inter-chunk
// product O1 = x1 state is pulled into registers and gated there; the intra-chunk product re-uses
// its TMEM columns, so no accumulator is written back.
// All waits are bounded; a timeout records an id in the unit's error word and every role drains out.
#include "tc.cuh"

FLAB_TC_DEFINE_ERROR_WORD(tc_chunk_o_error)

namespace flab {

enum { TMODE_O = 0, TMODE_DV = 1, TMODE_DV_LOCAL = 2 };

struct TcOParams {
  flab_args a;
  int n_items;   // NT * H * (V / BV)
  int v_tiles;   // V / BV
  int ab_fmt;    // 1 bf16, 0 fp16
};

template <int KB /*K/64*/, int VB /*BV/64*/, int MODE, int NS /*smem stages*/>
__global__ void __launch_bounds__(608, 1)
tc_chunk_o_kernel(const __grid_constant__ CUtensorMap mapX1, const __grid_constant__ CUtensorMap mapX2,
                  const __grid_constant__ CUtensorMap mapY, const __grid_constant__ CUtensorMap mapH,
                  const __grid_constant__ CUtensorMap mapOut, const TcOParams p) {
  using namespace tc;
  constexpr int K = 64 * KB, BV = 64 * VB;
  constexpr bool HAS_H = MODE != TMODE_DV_LOCAL;
  constexpr uint32_t X_BYTES = KB * 8192, Y_BYTES = VB * 8192, H_BYTES = HAS_H ? VB * K * 128 : 0;
  constexpr uint32_t STAGE_BYTES = 2 * X_BYTES + Y_BYTES + H_BYTES;
  constexpr uint32_t TM_STAGE = 256, TM_S = 0, TM_O = 64;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sStage = base;                         // [NS][STAGE_BYTES]
  unsigned char *sP = sStage + NS * STAGE_BYTES;         // [2][8192] score tiles (swizzled K-major)
  unsigned char *sOutAll = sP + 2 * 8192;                   // [2][VB][64][128 B] output tiles (swizzled, source of the tile store)
  float *sG = reinterpret_cast<float *>(sOutAll + 2 * Y_BYTES);  // [4][64]: gates of item i in slot i & 3
  __shared__ uint64_t full[NS], empty[NS], fullY[NS], emptyY[NS], s_done[2], p_ready[2], o_done[2], t_free[2];
  __shared__ uint64_t gates_full[4], gates_free[4], out_ready[2], out_free[2], copy_done[2];
  __shared__ int sRows[4];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const flab_args &a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&fullY[i], 1);
      mbar_init(&emptyY[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_done[i], 1);
      mbar_init(&p_ready[i], 8);
      mbar_init(&o_done[i], 1);
      mbar_init(&t_free[i], 8);
      mbar_init(&out_ready[i], 8);
      mbar_init(&out_free[i], 1);
      mbar_init(&copy_done[i], 8);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&gates_full[i], 1);
      mbar_init(&gates_free[i], 8);
    }
    abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const bool use_g = a.g != nullptr;
  const int n_local = p.n_items > (int)blockIdx.x ? (p.n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  auto fail = [&](int code) {
    abort_flag = 1;
    atomicCAS(&tu_tc_error, 0, code);
  };
  // item -> (chunk, head, v tile)
  auto decode = [&](int item, int &c, int &hd, int &vt) {
    vt = item % p.v_tiles;
    const int ch = item / p.v_tiles;
    hd = ch % a.H;
    c = ch / a.H;
  };

  if (warp == 16) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        const int st = i % NS, ph = (i / NS) & 1;
        // (where the item lies is worked out before the wait: the loads go out the moment the stage is free)
        int c, hd, vt, n, it;
        decode(blockIdx.x + i * gridDim.x, c, hd, vt);
        chunk_of(a, c, n, it);
        const Seq s = seq_of(a, n);
        const int t0 = s.bos + it * C;
        if (!mbar_wait(&empty[st], ph ^ 1)) { fail(1); break; }  // x1 | x2 | state of the stage's previous item are dead
        unsigned char *x1 = sStage + st * STAGE_BYTES, *x2 = x1 + X_BYTES, *y = x2 + X_BYTES, *hh = y + Y_BYTES;
        mbar_expect_tx(&full[st], STAGE_BYTES - Y_BYTES);
        const int c1 = a.head_first ? t0 : hd, c2 = a.head_first ? hd : t0;
#pragma unroll
        for (int j = 0; j < KB; ++j) {
          tma_load_4d(x1 + j * 8192, &mapX1, &full[st], 64 * j, c1, c2, s.b);
          tma_load_4d(x2 + j * 8192, &mapX2, &full[st], 64 * j, c1, c2, s.b);
        }
        if (HAS_H) {
#pragma unroll
          for (int j = 0; j < VB; ++j) tma_load_2d(hh + j * (K * 128), &mapH, &full[st], vt * BV + 64 * j, ((s.c0 + it) * a.H + hd) * K);
        }
        if (!mbar_wait(&emptyY[st], ph ^ 1)) { fail(13); break; }  // the last product of the stage's previous item has read y
        mbar_expect_tx(&fullY[st], Y_BYTES);
#pragma unroll
        for (int j = 0; j < VB; ++j) tma_load_4d(y + j * 8192, &mapY, &fullY[st], vt * BV + 64 * j, c1, c2, s.b);
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(64, 64, p.ab_fmt, 0, 0);
      const uint32_t idesc_h = instr_desc(64, BV, p.ab_fmt, 0, 1);
      auto issue12 = [&](int i) -> bool {
        const int st = i % NS, ph = (i / NS) & 1, ts = i & 1, tph = (i >> 1) & 1;
        if (!mbar_wait(&full[st], ph)) { fail(2); return false; }
        if (!mbar_wait(&t_free[ts], tph ^ 1)) { fail(3); return false; }
        fence_after_sync();
        const uint32_t x1 = smem_u32(sStage + st * STAGE_BYTES), x2 = x1 + X_BYTES, hh = x2 + X_BYTES + Y_BYTES;
        const uint32_t t = tmem + ts * TM_STAGE;
#pragma unroll
        for (int s = 0; s < 4 * KB; ++s) umma(t + TM_S, desc_kmajor(x1, s, 8192), desc_kmajor(x2, s, 8192), idesc_s, s > 0);
        if (HAS_H) {
#pragma unroll
          for (int s = 0; s < 4 * KB; ++s) umma(t + TM_O, desc_kmajor(x1, s, 8192), desc_mnmajor(hh, s, K * 128), idesc_h, s > 0);
        }
        umma_commit(&s_done[ts]);
        umma_commit(&empty[st]);  // x1 | x2 | state may be refilled
        return true;
      };
      bool ok = n_local > 0 ? issue12(0) : true;
      for (int i = 0; i < n_local && ok && !abort_flag; ++i) {
        const int st = i % NS, ts = i & 1, tph = (i >> 1) & 1;
        if (i + 1 < n_local) ok = issue12(i + 1);
        if (!ok) break;
        if (!mbar_wait(&p_ready[ts], tph)) { fail(4); break; }
        if (!mbar_wait(&fullY[st], (i / NS) & 1)) { fail(14); break; }
        fence_after_sync();
        const uint32_t y = smem_u32(sStage + st * STAGE_BYTES) + 2 * X_BYTES, pp = smem_u32(sP + ts * 8192);
        const uint32_t t = tmem + ts * TM_STAGE;
#pragma unroll
        for (int s = 0; s < 4; ++s) umma(t + TM_O, desc_kmajor(pp, s, 8192), desc_mnmajor(y, s, 8192), idesc_h, s > 0);
        umma_commit(&o_done[ts]);
        umma_commit(&emptyY[st]);
      }
    }
  } else if (warp == 18) {
    // ------------------------------------------------------------------ scalar warp
    // The gates of item i + 1 are fetched into registers before item i is published, so that the latency of the global
    // loads never limits how fast slots are filled (a short item lasts about as long as one such load).
    auto fetch = [&](int i, float &g0, float &g1, int &rows) {
      g0 = g1 = 0.f;
      rows = 0;
      if (i >= n_local) return;
      int c, hd, vt, n, it;
      decode(blockIdx.x + i * gridDim.x, c, hd, vt);
      chunk_of(a, c, n, it);
      const Seq s = seq_of(a, n);
      const int t0 = it * C;
      rows = min(C, s.len - t0);
      if (use_g) {
        const float *G = reinterpret_cast<const float *>(a.g);
        if (lane < rows) g0 = G[tok_off(a, s, hd, t0 + lane, 1)];
        if (lane + 32 < rows) g1 = G[tok_off(a, s, hd, t0 + lane + 32, 1)];
      }
    };
    // Lane 0 also sends the finished output tiles on their way, three items behind the gates it publishes: it waits for
    // the eight warps of the item's group, issues the tile stores and, once the copy engine has read the PREVIOUS item's
    // tile (or, after a ragged chunk, once that group's warps have copied their rows out), tells the other group that
    // its output buffer is free.  No epilogue warp issues a store or waits for one.
    int n_rag0 = 0, n_rag1 = 0;  // ragged items seen per group
    int prev_rows = C;  // row count of the item before the one being stored
    auto store_out = [&](int j) -> bool {
      const int grp = j & 1, kk = j >> 1;
      if (!mbar_wait(&out_ready[grp], kk & 1)) { fail(10); return false; }
      int c, hd, vt, n, it;
      decode(blockIdx.x + j * gridDim.x, c, hd, vt);
      chunk_of(a, c, n, it);
      const Seq s = seq_of(a, n);
      const int rows = min(C, s.len - it * C);
      if (rows == C) {
        const int tt = s.bos + it * C, c1 = a.head_first ? tt : hd, c2 = a.head_first ? hd : tt;
        unsigned char *src = sOutAll + grp * Y_BYTES;
#pragma unroll
        for (int jj = 0; jj < VB; ++jj) tma_store_4d(&mapOut, src + jj * 8192, vt * BV + 64 * jj, c1, c2, s.b);
        tma_store_commit();
      }
      if (j >= 1) {
        const int og = grp ^ 1;
        if (prev_rows < C) {
          if (!mbar_wait(&copy_done[og], (og ? n_rag1 : n_rag0) & 1)) { fail(11); return false; }
          if (og) ++n_rag1;
          else ++n_rag0;
        } else if (rows == C) {
          tma_store_wait_read_but_one();
        } else {
          tma_store_wait_read();
        }
        mbar_arrive(&out_free[og]);
      }
      prev_rows = rows;
      return true;
    };
    float c0, c1, n0, n1;
    int crows, nrows;
    fetch(0, c0, c1, crows);
    bool alive = true;
    for (int i = 0; i < n_local && alive && !abort_flag; ++i) {
      const int slot = i & 3;
      fetch(i + 1, n0, n1, nrows);
      if (i >= 4 && !mbar_wait(&gates_free[slot], ((i - 4) >> 2) & 1)) { fail(9); break; }  // item i - 4 has read the slot
      sG[slot * C + lane] = c0;
      sG[slot * C + lane + 32] = c1;
      if (lane == 0) sRows[slot] = crows;
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&gates_full[slot]);
        if (i >= 3) alive = store_out(i - 3);
      }
      alive = __shfl_sync(0xffffffffu, alive, 0);
      c0 = n0, c1 = n1, crows = nrows;
    }
    if (lane == 0) {
      for (int j = n_local > 3 ? n_local - 3 : 0; j < n_local && alive && !abort_flag; ++j) alive = store_out(j);
      tma_store_wait_all();
    }
  } else {
    // ------------------------------------------------------------------ epilogue groups (warps 0-7, 8-15)
    const int grp = warp >> 3, gw = warp & 7, wq = gw & 3, chh = gw >> 2, etid = tid & 255;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int m0 = wq * 16;
    const uint32_t lane_base = (uint32_t)(32 * wq) << 16;
    constexpr int NIO = 4 * VB;  // accumulator n-tiles of this warp's half of the O columns
    unsigned char *sOut = sOutAll + grp * Y_BYTES;
    const int row_lo = m0 + g8, row_hi = row_lo + 8;
    for (int i = grp; i < n_local && !abort_flag; i += 2) {
      const int st = grp, ph = (i >> 1) & 1, k = i >> 1, slot = i & 3;
      // gates and row count of this item, from the scalar warp
      if (!mbar_wait(&gates_full[slot], (i >> 2) & 1)) { fail(7); break; }
      const int rows = sRows[slot], last = rows - 1;
      float *gs = sG + slot * C;
      if (!mbar_wait(&s_done[st], ph)) { fail(5); break; }
      fence_after_sync();
      const uint32_t t = tmem + st * TM_STAGE + lane_base;
      const float g_lo = gs[row_lo], g_hi = gs[row_hi];
      // ---- S -> P : this warp's 16 rows x 32 columns
      {
        float sc[4][4];
        tmem_ld_frag<4>(t + TM_S + 32 * chh, sc);
        tmem_ld_wait();
        unsigned char *pp = sP + st * 8192;
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
          const int col = 32 * chh + 8 * ni + 2 * t4;
          const float gc0 = gs[col], gc1 = gs[col + 1];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int row = hf ? row_hi : row_lo;
            const float gr = hf ? g_hi : g_lo;
            float x0 = sc[ni][2 * hf], x1 = sc[ni][2 * hf + 1];
            if (MODE == TMODE_O) {
              x0 = (row >= col) ? (use_g ? x0 * __expf(fminf(gr - gc0, 0.f)) : x0) : 0.f;
              x1 = (row >= col + 1) ? (use_g ? x1 * __expf(fminf(gr - gc1, 0.f)) : x1) : 0.f;
            } else {
              x0 = (row <= col && col < rows) ? (use_g ? x0 * __expf(fminf(gc0 - gr, 0.f)) : x0) * a.scale : 0.f;
              x1 = (row <= col + 1 && col + 1 < rows) ? (use_g ? x1 * __expf(fminf(gc1 - gr, 0.f)) : x1) * a.scale : 0.f;
            }
            const uint32_t off = (uint32_t)row * 128u + ((uint32_t)((4 * chh + ni) ^ (row & 7)) << 4) + 4u * t4;
            if (p.ab_fmt) *reinterpret_cast<__nv_bfloat162 *>(pp + off) = __floats2bfloat162_rn(x0, x1);
            else *reinterpret_cast<__half2 *>(pp + off) = __floats2half2_rn(x0, x1);
          }
        }
      }
      // ---- O1 = x1 state -> registers, gated : 16 rows x BV/2 columns
      float o1[NIO][4];
      if (HAS_H) {
        tmem_ld_frag<NIO>(t + TM_O + (BV / 2) * chh, o1);
        tmem_ld_wait();
        if (use_g) {
          float s_lo, s_hi;
          if (MODE == TMODE_O) {
            s_lo = __expf(g_lo);
            s_hi = __expf(g_hi);
          } else {
            s_lo = __expf(fminf(gs[last] - g_lo, 0.f));
            s_hi = __expf(fminf(gs[last] - g_hi, 0.f));
          }
#pragma unroll
          for (int ni = 0; ni < NIO; ++ni) {
            o1[ni][0] *= s_lo;
            o1[ni][1] *= s_lo;
            o1[ni][2] *= s_hi;
            o1[ni][3] *= s_hi;
          }
        }
      }
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&p_ready[st]);
        mbar_arrive(&gates_free[slot]);  // this warp has read the item's gates for the last time
      }
      // ---- O2 = P y
      if (!mbar_wait(&o_done[st], ph)) { fail(6); break; }
      fence_after_sync();
      float o2[NIO][4];
      tmem_ld_frag<NIO>(t + TM_O + (BV / 2) * chh, o2);
      tmem_ld_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&t_free[st]);
      // the group's previous tile has left sOut (the scalar warp says so)
      if (k >= 1 && !mbar_wait(&out_free[grp], (k - 1) & 1)) { fail(8); break; }
      const float osc = MODE == TMODE_O ? a.scale : 1.f;
#pragma unroll
      for (int ni = 0; ni < NIO; ++ni)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int row = hf ? row_hi : row_lo, col = (BV / 2) * chh + 8 * ni + 2 * t4;
          const float x0 = (o2[ni][2 * hf] + (HAS_H ? o1[ni][2 * hf] : 0.f)) * osc;
          const float x1 = (o2[ni][2 * hf + 1] + (HAS_H ? o1[ni][2 * hf + 1] : 0.f)) * osc;
          unsigned char *dst = sOut + (col >> 6) * 8192 + sw128_offset(row, col & 63);
          if (p.ab_fmt) *reinterpret_cast<__nv_bfloat162 *>(dst) = __floats2bfloat162_rn(x0, x1);
          else *reinterpret_cast<__half2 *>(dst) = __floats2half2_rn(x0, x1);
        }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&out_ready[grp]);  // this warp's part of the output tile is written
      if (rows < C) {
        // ragged last chunk of a sequence: a tile store would write past its end; once the whole tile is there the
        // group's warps copy the valid rows out with ordinary stores
        if (!mbar_wait(&out_ready[grp], k & 1)) { fail(12); break; }
        int c, hd, vt, n, it;
        decode(blockIdx.x + i * gridDim.x, c, hd, vt);
        chunk_of(a, c, n, it);
        const Seq s = seq_of(a, n);
        const int t0 = it * C;
        bf16 *out = reinterpret_cast<bf16 *>(MODE == TMODE_O ? a.o : a.dv) + tok_off(a, s, hd, t0, a.V) + vt * BV;
        const size_t vs = tok_stride(a, a.V);
        for (int e = etid; e < rows * (BV / 8); e += 256) {
          const int r_ = e / (BV / 8), c_ = (e - r_ * (BV / 8)) * 8;
          *reinterpret_cast<int4 *>(out + (size_t)r_ * vs + c_) = *reinterpret_cast<const int4 *>(sOut + (c_ >> 6) * 8192 + sw128_offset(r_, c_ & 63));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&copy_done[grp]);
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <int KB, int VB, int MODE, int NS> static int launch_tc_o(const flab_args *a, cudaStream_t stream, const char *name) {
  constexpr int K = 64 * KB, BV = 64 * VB;
  CUtensorMap mX1, mX2, mY, mH, mOut;
  const void *x1 = MODE == TMODE_O ? a->q : a->k, *x2 = MODE == TMODE_O ? a->k : a->q;
  const void *y = MODE == TMODE_O ? a->v : a->d_o, *hs = MODE == TMODE_O ? a->h : a->dh;
  if (int e = make_token_map(&mX1, x1, a, a->K)) return e;
  if (int e = make_token_map(&mX2, x2, a, a->K)) return e;
  if (int e = make_token_map(&mY, y, a, a->V)) return e;
  if (MODE != TMODE_DV_LOCAL) {
    if (int e = make_state_map(&mH, hs, a, K)) return e;
  } else {
    mH = mY;
  }
  if (int e = make_token_map(&mOut, MODE == TMODE_O ? a->o : a->dv, a, a->V)) return e;
  TcOParams p;
  p.a = *a;
  p.v_tiles = a->V / BV;
  p.n_items = a->NT * a->H * p.v_tiles;
  p.ab_fmt = a->dtype == FLAB_BF16 ? 1 : 0;
  constexpr uint32_t STAGE = 2 * KB * 8192 + VB * 8192 + (MODE != TMODE_DV_LOCAL ? VB * K * 128 : 0);
  const size_t smem = 1024 + NS * (size_t)STAGE + 2 * 8192 + 2 * (size_t)VB * 8192 + 4 * C * sizeof(float);
  auto kern = tc_chunk_o_kernel<KB, VB, MODE, NS>;
  if (int e = set_smem(kern, smem)) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.n_items < sms ? p.n_items : sms;
  kern<<<grid, 608, smem, stream>>>(mX1, mX2, mY, mH, mOut, p);
  return check_launch(name);
}

// Returns 1 if the tcgen05 kernel took the call, 0 if the shape is outside its domain, < 0 on error.
template <int MODE> int tc_chunk_o_try(const flab_args *a, cudaStream_t stream, const char *name) {
  if (a->dtype != FLAB_BF16 && a->dtype != FLAB_FP16) return 0;
  if ((a->K != 64 && a->K != 128) || a->V % 64 != 0) return 0;
  if ((unsigned long long)a->NT * a->H * a->K >= (1ull << 31)) return 0;  // tile coordinates of the state tensor are 32-bit
  const void *ptrs[5] = {a->q, a->k, MODE == TMODE_O ? a->v : a->d_o, MODE == TMODE_O ? a->h : (MODE == TMODE_DV ? a->dh : a->q),
                         MODE == TMODE_O ? a->o : a->dv};
  for (int i = 0; i < 5; ++i)
    if (reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return 0;
  // shared-memory stages: as many as fit next to the two score tiles and the two staging buffers
  constexpr bool L = MODE == TMODE_DV_LOCAL;
  int rc;
  if (a->K == 64) {
    rc = (a->V % 128 == 0) ? launch_tc_o<1, 2, MODE, L ? 4 : 3>(a, stream, name) : launch_tc_o<1, 1, MODE, 4>(a, stream, name);  // (1, 2) with four stages and a state tile is 241 KB
  } else {
    rc = (a->V % 128 == 0) ? launch_tc_o<2, 2, MODE, L ? 3 : 2>(a, stream, name) : launch_tc_o<2, 1, MODE, L ? 4 : 3>(a, stream, name);
  }
  return rc < 0 ? rc : 1;
}

template int tc_chunk_o_try<TMODE_O>(const flab_args *, cudaStream_t, const char *);
template int tc_chunk_o_try<TMODE_DV>(const flab_args *, cudaStream_t, const char *);
template int tc_chunk_o_try<TMODE_DV_LOCAL>(const flab_args *, cudaStream_t, const char *);

}  // namespace flab
