// tcgen05 / TMA version of chunk_bwd_dqkwg (bf16 / fp16, K = V = 128):
//   dq = scale e^{b_i} (do h^T) + ds k            ds = tril(do v^T * e^{b_i-b_j}) * scale
//   dk = e^{b_L-b_j} (v dh^T) + ds^T q
//   dw = -e^{b_i} (dv h^T)                         (delta-rule families only)
//   dg_i = <q_i, dq_i> - <k_i, dk_i> + <w_i, dw_i>;  dg_last += e^{b_L} <h, dh> + <k, dk_inter>
//   (fla/ops/common/chunk_o.py:444-600)
// Persistent kernel, one CTA per SM, work item = (chunk, head).  Twenty warps:
//   warp 16 : TMA producer - X1 = {do, v, dv} (48 KB, two buffers), X2 = {h, dh} (64 KB, one buffer) and
//             Y = {q, k, w} (48 KB, one buffer).  The item starts on X1 (ds, row factors), so X1 of the next item
//             is fetched a whole item ahead; X2 is refilled as soon as the products against the states are done,
//             Y as soon as the last phase has read q, k, w.  The outputs are built over the item's own do, v, dv tiles
//             (dead once the products against the states have run), so the tile store holds up only a buffer that is
//             not needed again for a whole item
//   warp 17 : MMA issuer   - ds = do v^T; then the three products against the states; then the two
//             intra-chunk products, accumulated onto dq and dk in TMEM
//   warps 0-15 : epilogue, warp = (TMEM lane quadrant = 16 tokens, 32-column group)
//   warp 18 : output     - tile stores of dq, dk, dw from the item's X1 buffer, then hands the buffer back to the producer
//   warp 19 : scalars    - gates and row count of the coming item into shared memory, zeroed dg rows, and the finished
//                          dg rows of past items out to global memory: the epilogue warps touch no global memory per
//                          token and meet each other only through the mbarriers of the phases
// The row factors of the inter-chunk terms of dq and dk are applied to the A operands in shared memory (do and v are
// rescaled in place after ds has been formed from the unscaled tiles), so that inter- and intra-chunk parts
// add up in one accumulator and TMEM holds ds | dq | dk | dw = 448 columns.  dq, dk, dw are written over the
// item's do, v, dv tiles and leave through tile stores.
// All waits are bounded; a timeout records an id in the unit's error word and the epilogue warps leave
// together at their next common barrier.
#include "tc.cuh"

FLAB_TC_DEFINE_ERROR_WORD(tc_dqkwg_error)

namespace flab {

struct TcDqParams {
  flab_args a;
  int n_items;  // NT * H
  int ab_fmt;   // 1 bf16, 0 fp16
};

struct TcDqMaps {
  CUtensorMap q, k, w, v, d_o, dv, h, dh, dq, dk, dw;
};

template <bool USE_DW>
__global__ void __launch_bounds__(640, 1) tc_dqkwg_kernel(const __grid_constant__ TcDqMaps m, const TcDqParams p) {
  using namespace tc;
  constexpr uint32_t T16 = 16384, T32 = 32768;
  constexpr uint32_t X1_BYTES = (USE_DW ? 3 : 2) * T16, X2_BYTES = 2 * T32, Y_BYTES = (USE_DW ? 3 : 2) * T16;
  constexpr uint32_t TM_DS = 0, TM_DQ = 64, TM_DK = 192, TM_DW = 320;
  constexpr int ET = 512;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sX1 = base;                       // [2][do | v | dv]
  unsigned char *sH = sX1 + 2 * X1_BYTES, *sDH = sH + T32;  // X2
  unsigned char *sY = sDH + T32;                   // [q | k | w]
  unsigned char *sDS = sY + Y_BYTES;               // [64][128 B]
  float *sG = reinterpret_cast<float *>(sDS + 8192);  // [2][64] gates
  // partial sums of the epilogue warps: plain stores into a slot per (item parity, column group or warp), no atomics;
  // the scalar warp adds them up when it writes the rows out
  float *sDG = sG + 2 * C;                            // [2][4][64] dg rows per column group
  float *sRed = sDG + 8 * C;                          // [2][2][16] <h, dh>, <k, dk_inter> per epilogue warp
  __shared__ uint64_t fullX1[2], emptyX1[2], fullX2, emptyX2, fullY, emptyY, ds_done, e1_done, dk_done, e1b_done, all_done, acc_free, out_ready;
  __shared__ uint64_t scal_full[2], rows_done[2], ragged_sync;
  __shared__ int sRows[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const flab_args &a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int j = 0; j < 2; ++j) {
      mbar_init(&fullX1[j], 1);
      mbar_init(&emptyX1[j], 1);
    }
    mbar_init(&fullX2, 1);
    mbar_init(&emptyX2, 17);  // the products against the states have completed + every epilogue warp is done with h, dh
    mbar_init(&fullY, 1);
    mbar_init(&emptyY, 16);  // every epilogue warp has read q, k, w for the last time
    mbar_init(&ds_done, 1);
    mbar_init(&e1_done, 16);
    mbar_init(&dk_done, 1);
    mbar_init(&e1b_done, 16);
    mbar_init(&all_done, 1);
    mbar_init(&acc_free, 16);
    mbar_init(&out_ready, 16);
    for (int j = 0; j < 2; ++j) {
      mbar_init(&scal_full[j], 1);
      mbar_init(&rows_done[j], 16);
    }
    mbar_init(&ragged_sync, 16);
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
  // item -> (global chunk index, head)
  auto decode = [&](int i, int &c, int &hd) {
    const int item = blockIdx.x + i * gridDim.x;
    hd = item % a.H;
    c = item / a.H;
  };

  if (warp == 16) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        const int ph = i & 1;
        int c, hd, n, it;
        decode(i, c, hd);
        chunk_of(a, c, n, it);
        const Seq s = seq_of(a, n);
        const int t0 = s.bos + it * C;
        const int c1 = a.head_first ? t0 : hd, c2 = a.head_first ? hd : t0;
        const int srow = ((s.c0 + it) * a.H + hd) * 128;
        const int xb = i & 1, xph = (i >> 1) & 1;
        unsigned char *sDo = sX1 + xb * X1_BYTES, *sV = sDo + T16, *sDv = sV + T16;
        if (!mbar_wait(&emptyX1[xb], xph ^ 1)) { fail(61); break; }
        mbar_expect_tx(&fullX1[xb], X1_BYTES);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_4d(sDo + j * 8192, &m.d_o, &fullX1[xb], 64 * j, c1, c2, s.b);
          tma_load_4d(sV + j * 8192, &m.v, &fullX1[xb], 64 * j, c1, c2, s.b);
          if (USE_DW) tma_load_4d(sDv + j * 8192, &m.dv, &fullX1[xb], 64 * j, c1, c2, s.b);
        }
        if (!mbar_wait(&emptyX2, ph ^ 1)) { fail(74); break; }
        mbar_expect_tx(&fullX2, X2_BYTES);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_2d(sH + j * T16, &m.h, &fullX2, 64 * j, srow);
          tma_load_2d(sDH + j * T16, &m.dh, &fullX2, 64 * j, srow);
        }
        unsigned char *sQ = sY, *sK = sQ + T16, *sW = sK + T16;
        if (!mbar_wait(&emptyY, ph ^ 1)) { fail(62); break; }
        mbar_expect_tx(&fullY, Y_BYTES);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_4d(sQ + j * 8192, &m.q, &fullY, 64 * j, c1, c2, s.b);
          tma_load_4d(sK + j * 8192, &m.k, &fullY, 64 * j, c1, c2, s.b);
          if (USE_DW) tma_load_4d(sW + j * 8192, &m.w, &fullY, 64 * j, c1, c2, s.b);
        }
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t id_ds = instr_desc(64, 64, p.ab_fmt, 0, 0);    // do v^T      : A, B K-major
      const uint32_t id_st = instr_desc(64, 128, p.ab_fmt, 0, 0);   // x state^T   : A, B K-major
      const uint32_t id_dq = instr_desc(64, 128, p.ab_fmt, 0, 1);   // ds k        : A K-major, B MN-major
      const uint32_t id_dk = instr_desc(64, 128, p.ab_fmt, 1, 1);   // ds^T q      : A, B MN-major
      const uint64_t d_h = desc_kmajor(smem_u32(sH), 0, T16), d_dh = desc_kmajor(smem_u32(sDH), 0, T16);
      const uint64_t d_dsk = desc_kmajor(smem_u32(sDS), 0, 8192), d_dsm = desc_mnmajor(smem_u32(sDS), 0, 8192);
      // per-step advance of the start-address field (16-byte units)
      auto kx = [](int k, uint32_t box) -> uint64_t { return (uint64_t)(((k >> 2) * box + (k & 3) * 32) >> 4); };
      auto mx = [](int k) -> uint64_t { return (uint64_t)((k * 2048) >> 4); };
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        const int ph = i & 1;
        const int xb = i & 1, xph = (i >> 1) & 1;
        const uint32_t x1 = smem_u32(sX1 + xb * X1_BYTES);
        const uint64_t d_do = desc_kmajor(x1, 0, 8192), d_v = desc_kmajor(x1 + T16, 0, 8192), d_dv = desc_kmajor(x1 + 2 * T16, 0, 8192);
        if (!mbar_wait(&fullX1[xb], xph)) { fail(63); break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma(tmem + TM_DS, d_do + kx(k, 8192), d_v + kx(k, 8192), id_ds, k > 0);
        umma_commit(&ds_done);
        if (!mbar_wait(&e1_done, ph)) { fail(64); break; }
        if (i > 0 && !mbar_wait(&acc_free, ph ^ 1)) { fail(65); break; }
        if (!mbar_wait(&fullX2, ph)) { fail(75); break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma(tmem + TM_DK, d_v + kx(k, 8192), d_dh + kx(k, T16), id_st, k > 0);
        umma_commit(&dk_done);  // the epilogue takes <k, dk_inter> from it while the other products run
#pragma unroll
        for (int k = 0; k < 8; ++k) umma(tmem + TM_DQ, d_do + kx(k, 8192), d_h + kx(k, T16), id_st, k > 0);
        if (USE_DW) {
#pragma unroll
          for (int k = 0; k < 8; ++k) umma(tmem + TM_DW, d_dv + kx(k, 8192), d_h + kx(k, T16), id_st, k > 0);
        }
        umma_commit(&emptyX2);
        const uint64_t d_q = desc_mnmajor(smem_u32(sY), 0, 8192), d_k = desc_mnmajor(smem_u32(sY + T16), 0, 8192);
        if (!mbar_wait(&fullY, ph)) { fail(66); break; }
        if (use_g && !mbar_wait(&e1b_done, ph)) { fail(67); break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_DQ, d_dsk + kx(k, 8192), d_k + mx(k), id_dq, 1);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_DK, d_dsm + mx(k), d_q + mx(k), id_dk, 1);
        umma_commit(&all_done);
      }
    }
  } else if (warp == 18) {
    // ------------------------------------------------------------------ output warp
    if (lane == 0) {
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        int c, hd, n, it;
        decode(i, c, hd);
        chunk_of(a, c, n, it);
        const Seq s = seq_of(a, n);
        const int t0 = it * C, rows = min(C, s.len - t0);
        const int xb = i & 1;
        unsigned char *oQ = sX1 + xb * X1_BYTES, *oK = oQ + T16, *oW = oK + T16;  // dq over do, dk over v, dw over dv
        if (!mbar_wait(&out_ready, i & 1)) { fail(73); break; }
        if (rows == C) {  // (a ragged chunk was written out by the epilogue warps themselves)
          const int tt = s.bos + t0, c1 = a.head_first ? tt : hd, c2 = a.head_first ? hd : tt;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            tma_store_4d(&m.dq, oQ + j * 8192, 64 * j, c1, c2, s.b);
            tma_store_4d(&m.dk, oK + j * 8192, 64 * j, c1, c2, s.b);
            if (USE_DW) tma_store_4d(&m.dw, oW + j * 8192, 64 * j, c1, c2, s.b);
          }
          tma_store_commit();
          tma_store_wait_read();
        }
        mbar_arrive(&emptyX1[xb]);
      }
      tma_store_wait_all();
    }
  } else if (warp == 19) {
    // ------------------------------------------------------------------ scalar warp
    // Item i uses slot i & 1 of sG / sDG / sRed / sRows.  A slot is handed to item i once item i - 2 is finished with
    // it (rows_done); its dg rows go to global memory from here, the chunk's last row with the two state terms added.
    const float *Gbase = reinterpret_cast<const float *>(a.g);
    auto where = [&](int j, Seq &s, int &hd, int &t0, int &rows) {
      int c, n, it;
      decode(j, c, hd);
      chunk_of(a, c, n, it);
      s = seq_of(a, n);
      t0 = it * C;
      rows = min(C, s.len - t0);
    };
    auto write_out = [&](int j) -> bool {
      const int slot = j & 1;
      if (!mbar_wait(&rows_done[slot], (j >> 1) & 1)) {
        fail(77);
        return false;
      }
      if (!use_g) return true;
      Seq s;
      int hd, t0, rows;
      where(j, s, hd, t0, rows);
      const float *gs = sG + slot * C, *dgs = sDG + slot * 4 * C, *red = sRed + slot * 32;
      float r0 = lane < 16 ? red[lane] : 0.f, r1 = lane < 16 ? red[16 + lane] : 0.f;  // the 16 warps' shares of the two state terms
      r0 = warp_sum(r0);
      r1 = warp_sum(r1);
      for (int t = lane; t < rows; t += 32) {
        float x = (dgs[t] + dgs[C + t]) + (dgs[2 * C + t] + dgs[3 * C + t]);
        if (t == rows - 1) x += r0 * __expf(gs[t]) + r1;
        reinterpret_cast<float *>(a.dg)[tok_off(a, s, hd, t0 + t, 1)] = x;
      }
      return true;
    };
    // the gates of item i + 1 are fetched into registers before item i is published and before the wait for item i - 2:
    // the latency of these global loads is never exposed
    auto fetch = [&](int i, float (&gt)[2], int &rows) {
      gt[0] = gt[1] = 0.f;
      rows = 0;
      if (i >= n_local) return;
      Seq s;
      int hd, t0;
      where(i, s, hd, t0, rows);
      if (use_g) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
          if (lane + 32 * h < rows) gt[h] = Gbase[tok_off(a, s, hd, t0 + lane + 32 * h, 1)];
      }
    };
    float cg[2], ng[2];
    int crows, nrows;
    fetch(0, cg, crows);
    bool alive = true;
    for (int i = 0; i < n_local && alive && !abort_flag; ++i) {
      const int slot = i & 1;
      fetch(i + 1, ng, nrows);
      if (i >= 2) alive = write_out(i - 2);
      __syncwarp();
      if (!alive) break;
      sG[slot * C + lane] = cg[0];
      sG[slot * C + lane + 32] = cg[1];
      if (lane == 0) sRows[slot] = crows;
      __syncwarp();
      if (lane == 0) mbar_arrive(&scal_full[slot]);
      cg[0] = ng[0], cg[1] = ng[1], crows = nrows;
    }
    for (int j = n_local > 2 ? n_local - 2 : 0; j < n_local && alive && !abort_flag; ++j) {
      alive = write_out(j);
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 0-15
    const int wq = warp & 3, cq = warp >> 2, g8 = lane >> 2, t4 = lane & 3;
    const uint32_t lane_base = (uint32_t)(32 * wq) << 16;
    const int row_lo = 16 * wq + g8, row_hi = row_lo + 8;
    const int colb = 32 * cq + 2 * t4;  // this thread's columns: colb + 8 ni (+1)
    // byte offsets of this thread's 16 element pairs inside a [2 boxes][64 tokens][128 B] tile
    uint32_t o_lo_[4], o_hi_[4];
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      const int col = colb + 8 * ni;
      o_lo_[ni] = (uint32_t)(col >> 6) * 8192u + sw128_offset(row_lo, col & 63);
      o_hi_[ni] = (uint32_t)(col >> 6) * 8192u + sw128_offset(row_hi, col & 63);
    }
    // packed 16-bit pair <-> floats in the kernel's element format
    auto ld2 = [&](const unsigned char *ptr) -> float2 {
      return p.ab_fmt ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(ptr))
                      : __half22float2(*reinterpret_cast<const __half2 *>(ptr));
    };
    auto st2 = [&](unsigned char *ptr, float x, float y) {
      if (p.ab_fmt) *reinterpret_cast<__nv_bfloat162 *>(ptr) = __floats2bfloat162_rn(x, y);
      else *reinterpret_cast<__half2 *>(ptr) = __floats2half2_rn(x, y);
    };
    int n_ragged = 0;
    for (int i = 0; i < n_local && !abort_flag; ++i) {
      const int ph = i & 1;
      const int xb = i & 1, xph = (i >> 1) & 1;
      // gates, row count and the zeroed dg rows / state terms of this item, from the scalar warp
      if (!mbar_wait(&scal_full[ph], xph)) fail(78);
      const int rows = sRows[ph], last = rows - 1;
      float *gs = sG + ph * C, *dgs = sDG + (ph * 4 + cq) * C, *red = sRed + ph * 32;
      unsigned char *sDo = sX1 + xb * X1_BYTES, *sV = sDo + T16, *sDv = sV + T16;
      unsigned char *sQ = sY, *sK = sQ + T16, *sW = sK + T16;
      const float g_lo = gs[row_lo], g_hi = gs[row_hi], gl = gs[last];
      const float e_lo = use_g ? __expf(g_lo) : 1.f, e_hi = use_g ? __expf(g_hi) : 1.f;
      const float f_lo = use_g ? __expf(fminf(gl - g_lo, 0.f)) : 1.f, f_hi = use_g ? __expf(fminf(gl - g_hi, 0.f)) : 1.f;
      // ---- E1: <h, dh>; ds -> masked / decayed operand; row factors onto do, v, dv
      if (!mbar_wait(&fullX1[xb], xph)) fail(68);
      if (!mbar_wait(&ds_done, ph)) fail(69);
      fence_after_sync();
      {
        // ds: all sixteen warps, 16 columns each
        float sc[2][4];
        tmem_ld_frag<2>(tmem + lane_base + TM_DS + 16 * cq, sc);
        tmem_ld_wait();
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
          const int col = 16 * cq + 8 * ni + 2 * t4;
          const float gc0 = gs[col], gc1 = gs[col + 1];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int row = hf ? row_hi : row_lo;
            const float gr = hf ? g_hi : g_lo;
            float x0 = sc[ni][2 * hf], x1 = sc[ni][2 * hf + 1];
            const bool v0 = row >= col && row < rows, v1 = row >= col + 1 && row < rows;
            x0 = v0 ? (use_g ? x0 * __expf(fminf(gr - gc0, 0.f)) : x0) * a.scale : 0.f;
            x1 = v1 ? (use_g ? x1 * __expf(fminf(gr - gc1, 0.f)) : x1) * a.scale : 0.f;
            st2(sDS + sw128_offset(row, col), x0, x1);
          }
        }
      }
      {
        // do' = scale e^{b} do and v' = e^{b_L-b} v, in place (ds was formed from the unscaled tiles); a row factor does
        // not care about the swizzle, so every thread rescales two whole 16-byte pieces of one token row per tile
        // (the factor of dw, -e^{b}, is applied to the fp32 accumulator at the end of the item instead)
        const int pr = tid >> 3;  // token row of this thread's pieces (one in each 64-column box)
        const float gp = gs[pr];
        const float sd = (use_g ? __expf(gp) : 1.f) * a.scale, fv = use_g ? __expf(fminf(gl - gp, 0.f)) : 1.f;
        auto rescale = [&](unsigned char *tile, float f) {
#pragma unroll
          for (int bx = 0; bx < 2; ++bx) {
            int4 *ptr = reinterpret_cast<int4 *>(tile + bx * 8192 + tid * 16);
            int4 x = *ptr;
            uint32_t *u = reinterpret_cast<uint32_t *>(&x);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f2 = ld2(reinterpret_cast<const unsigned char *>(&u[e]));
              st2(reinterpret_cast<unsigned char *>(&u[e]), f2.x * f, f2.y * f);
            }
            *ptr = x;
          }
        };
        rescale(sDo, sd);
        if (use_g) rescale(sV, fv);
      }
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&e1_done);
      // <h, dh> while the tensor core works; then this warp is done with the state tiles
      if (use_g) {
        if (!mbar_wait(&fullX2, ph)) fail(76);
        float hd_ = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int idx = tid + ET * j;  // 16-byte piece of the [2 boxes][128 rows][8 pieces] tiles
          const int4 xa = *reinterpret_cast<const int4 *>(sH + idx * 16), xb = *reinterpret_cast<const int4 *>(sDH + idx * 16);
          const uint32_t *ua = reinterpret_cast<const uint32_t *>(&xa), *ub = reinterpret_cast<const uint32_t *>(&xb);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 fa = ld2(reinterpret_cast<const unsigned char *>(&ua[e])), fb = ld2(reinterpret_cast<const unsigned char *>(&ub[e]));
            hd_ = fmaf(fa.x, fb.x, fmaf(fa.y, fb.y, hd_));
          }
        }
        hd_ = warp_sum(hd_);
        if (lane == 0) red[warp] = hd_;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&emptyX2);
      // ---- E1b: <k, dk_inter> from the inter-chunk dk before the intra-chunk product lands on it
      if (!mbar_wait(&fullY, ph)) fail(70);
      if (use_g) {
        if (!mbar_wait(&dk_done, ph)) fail(71);
        fence_after_sync();
        float dki[4][4];
        tmem_ld_frag<4>(tmem + lane_base + TM_DK + 32 * cq, dki);
        tmem_ld_wait();
        float dkk = 0.f;
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
          const int col = colb + 8 * ni;
          const uint32_t o_lo = o_lo_[ni], o_hi = o_hi_[ni];
          const float2 k_lo = ld2(sK + o_lo), k_hi = ld2(sK + o_hi);
          if (row_lo < rows) dkk += dki[ni][0] * k_lo.x + dki[ni][1] * k_lo.y;
          if (row_hi < rows) dkk += dki[ni][2] * k_hi.x + dki[ni][3] * k_hi.y;
        }
        dkk = warp_sum(dkk);
        if (lane == 0) red[16 + warp] = dkk;
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&e1b_done);
      }
      // ---- E2: finished dq, dk, dw -> dg rows (dots with q, k, w), outputs over the item's do, v, dv tiles
      if (!mbar_wait(&all_done, ph)) fail(72);
      fence_after_sync();
      float dq[4][4], dk[4][4], dw[4][4];
      tmem_ld_frag<4>(tmem + lane_base + TM_DQ + 32 * cq, dq);
      tmem_ld_frag<4>(tmem + lane_base + TM_DK + 32 * cq, dk);
      if (USE_DW) tmem_ld_frag<4>(tmem + lane_base + TM_DW + 32 * cq, dw);
      tmem_ld_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free);
      float dg_lo = 0.f, dg_hi = 0.f;
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int col = colb + 8 * ni;
        const uint32_t o_lo = o_lo_[ni], o_hi = o_hi_[ni];
        if (use_g) {
          const float2 q_lo = ld2(sQ + o_lo), q_hi = ld2(sQ + o_hi), k_lo = ld2(sK + o_lo), k_hi = ld2(sK + o_hi);
          dg_lo += dq[ni][0] * q_lo.x + dq[ni][1] * q_lo.y - dk[ni][0] * k_lo.x - dk[ni][1] * k_lo.y;
          dg_hi += dq[ni][2] * q_hi.x + dq[ni][3] * q_hi.y - dk[ni][2] * k_hi.x - dk[ni][3] * k_hi.y;
        }
        st2(sDo + o_lo, dq[ni][0], dq[ni][1]);
        st2(sDo + o_hi, dq[ni][2], dq[ni][3]);
        st2(sV + o_lo, dk[ni][0], dk[ni][1]);
        st2(sV + o_hi, dk[ni][2], dk[ni][3]);
        if (USE_DW) {
          // dw = -e^{b} (dv h^T): the row factor goes onto the fp32 product here (dv itself was left as loaded)
          dw[ni][0] *= -e_lo, dw[ni][1] *= -e_lo, dw[ni][2] *= -e_hi, dw[ni][3] *= -e_hi;
          if (use_g) {
            const float2 w_lo = ld2(sW + o_lo), w_hi = ld2(sW + o_hi);
            dg_lo += dw[ni][0] * w_lo.x + dw[ni][1] * w_lo.y;
            dg_hi += dw[ni][2] * w_hi.x + dw[ni][3] * w_hi.y;
          }
          st2(sDv + o_lo, dw[ni][0], dw[ni][1]);
          st2(sDv + o_hi, dw[ni][2], dw[ni][3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&emptyY);  // q, k, w have been read for the last time: the producer may fetch the next item's
      if (use_g) {
        dg_lo += __shfl_xor_sync(0xffffffffu, dg_lo, 1);
        dg_lo += __shfl_xor_sync(0xffffffffu, dg_lo, 2);
        dg_hi += __shfl_xor_sync(0xffffffffu, dg_hi, 1);
        dg_hi += __shfl_xor_sync(0xffffffffu, dg_hi, 2);
        if (t4 == 0) {
          dgs[row_lo] = dg_lo;
          dgs[row_hi] = dg_hi;
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&rows_done[ph]);  // this warp's share of the dg rows and state terms is in shared memory
      if (rows < C) {
        // ragged last chunk of a sequence: a tile store would write past its end, so the epilogue warps copy the valid
        // rows themselves once every warp has finished its part of the output tiles
        if (lane == 0) mbar_arrive(&ragged_sync);
        if (!mbar_wait(&ragged_sync, n_ragged & 1)) fail(79);
        ++n_ragged;
        int c, hd, n, it;
        decode(i, c, hd);
        chunk_of(a, c, n, it);
        const Seq s = seq_of(a, n);
        const int t0 = it * C;
        const size_t ks = tok_stride(a, a.K), off0 = tok_off(a, s, hd, t0, a.K);
        for (int e = tid; e < rows * 16; e += ET) {
          const int r_ = e >> 4, c_ = (e & 15) * 8;
          const uint32_t so = (uint32_t)(c_ >> 6) * 8192u + sw128_offset(r_, c_ & 63);
          const size_t go = off0 + (size_t)r_ * ks + c_;
          *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.dq) + go) = *reinterpret_cast<const int4 *>(sDo + so);
          *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.dk) + go) = *reinterpret_cast<const int4 *>(sV + so);
          if (USE_DW) *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.dw) + go) = *reinterpret_cast<const int4 *>(sDv + so);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&out_ready);  // this warp's part of the output tiles is complete
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <bool USE_DW> static int launch_tc_dqkwg(const flab_args *a, cudaStream_t stream) {
  TcDqMaps m;
  if (int e = make_token_map(&m.q, a->q, a, a->K)) return e;
  if (int e = make_token_map(&m.k, a->k, a, a->K)) return e;
  if (int e = make_token_map(&m.w, USE_DW ? a->w : a->k, a, a->K)) return e;
  if (int e = make_token_map(&m.v, a->v, a, a->V)) return e;
  if (int e = make_token_map(&m.d_o, a->d_o, a, a->V)) return e;
  if (int e = make_token_map(&m.dv, USE_DW ? a->dv : a->v, a, a->V)) return e;
  if (int e = make_state_map(&m.h, a->h, a, 128)) return e;
  if (int e = make_state_map(&m.dh, a->dh, a, 128)) return e;
  if (int e = make_token_map(&m.dq, a->dq, a, a->K)) return e;
  if (int e = make_token_map(&m.dk, a->dk, a, a->K)) return e;
  if (int e = make_token_map(&m.dw, USE_DW ? a->dw : a->dk, a, a->K)) return e;
  TcDqParams p;
  p.a = *a;
  p.n_items = a->NT * a->H;
  p.ab_fmt = a->dtype == FLAB_BF16 ? 1 : 0;
  const size_t smem = 1024 + (size_t)(USE_DW ? 9 : 6) * 16384 + 2 * 32768 + 8192 + (10 * C + 64) * sizeof(float);
  auto kern = tc_dqkwg_kernel<USE_DW>;
  if (int e = set_smem(kern, smem)) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.n_items < sms ? p.n_items : sms;
  kern<<<grid, 640, smem, stream>>>(m, p);
  return check_launch("chunk_bwd_dqkwg(tc)");
}

// Returns 1 if the tcgen05 kernel took the call, 0 if the shape is outside its domain, < 0 on error.
int tc_dqkwg_try(const flab_args *a, cudaStream_t stream) {
  if (a->dtype != FLAB_BF16 && a->dtype != FLAB_FP16) return 0;
  if (a->K != 128 || a->V != 128) return 0;
  if ((unsigned long long)a->NT * a->H * a->K >= (1ull << 31)) return 0;  // tile coordinates of the state tensor are 32-bit
  const void *ptrs[11] = {a->q, a->k, a->w, a->v, a->d_o, a->dv, a->h, a->dh, a->dq, a->dk, a->dw};
  for (int i = 0; i < 11; ++i)
    if (ptrs[i] && reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return 0;
  const int rc = a->w ? launch_tc_dqkwg<true>(a, stream) : launch_tc_dqkwg<false>(a, stream);
  return rc < 0 ? rc : 1;
}

}  // namespace flab
