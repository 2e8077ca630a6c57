// tcgen05 / TMA version of the backward of the WY / UT transform (bf16 / fp16, K = V = 128):
//   given dw, du and the stored A matrices, with x in {k, v}, dx in {dw, du}:
//     dA_x  = strict_lower((dx x^T) diag(beta));   d(beta x) = A_x^T dx  ->  dx_out = d(beta x) beta,
//     dbeta += rowsum(d(beta x) * x);   dA_x <- -strict_lower(A_x^T dA_x A_x^T)
//   dA = dA_w + dA_u * e^{b_i-b_j}  (gated; ungated: one A, dA_w and dA_u are summed before the transform)
//   dk = (A_w^T dw) beta + (dA k) beta + (diag(beta) dA)^T k [+ dk of the preceding stage];
//   dbeta += rowsum((dA k) * k);   dg = rowsum(P) - colsum(P),  P = dA_u e^{b_i-b_j} * (diag(beta) k k^T)
//   (fla/ops/delta_rule/wy_fast.py:325-433, fla/ops/gated_delta_rule/wy_fast.py:440-562)
// Persistent kernel, one CTA per SM, work item = (chunk, head).  Twenty warps:
//   warp 16 : TMA producer - k, v, dw, du, dk_in, A_w, A_u of an item (96 KB), two buffers
//   warp 17 : MMA issuer   - four batches of products per item, accumulators in TMEM (512 columns, re-used)
//   warp 18 : output       - tile stores of dk and dv, which the epilogue builds over the dw and du tiles
//   warp 19 : scalars      - beta, gate and row count of the coming item into shared memory, zeroed dbeta / dg rows,
//                            and the finished dbeta / dg rows of past items out to global memory: every global load,
//                            global store and index computation per token is kept off the epilogue warps
//   warps 0-15 : epilogue, warp = (TMEM lane quadrant = 16 tokens, column group); the warps are tied to each other
//                            only through the mbarriers of the phases, never through a CTA-wide barrier
// Batches:  B1: dw k^T, A_w^T dw, du v^T, A_u^T du      E1: mask / beta / round -> dA operands; dv; dbeta
//           B2: dA_w A_w^T, dA_u A_u^T                  E2: round -> operands
//           B3: A_w^T (.), A_u^T (.)                    E3: sign, mask, decay, sum -> dA, diag(beta) dA
//           (k k^T behind B3)                           dbeta / dg sums over dA * k k^T
//           B4: (beta dA) k + (beta dA)^T k             E4: dk, dbeta
// All waits are bounded; a timeout records an id in the unit's error word and the epilogue warps leave
// together at their next common barrier.
#include "tc.cuh"

FLAB_TC_DEFINE_ERROR_WORD(tc_wy_bwd_error)

namespace flab {

struct TcWyParams {
  flab_args a;
  int n_items;  // NT * H
  int ab_fmt;   // 1 bf16, 0 fp16
};

struct TcWyMaps {
  CUtensorMap k, v, dw, du, dkin, aw, au, dk, dv;
};

template <bool GATED>
__global__ void __launch_bounds__(640, 1) tc_wy_bwd_kernel(const __grid_constant__ TcWyMaps m, const TcWyParams p) {
  using namespace tc;
  constexpr uint32_t T16 = 16384, T8 = 8192;
  constexpr uint32_t IN_BYTES = 5 * T16 + 2 * T8;  // one item's tiles
  // TMEM columns (fp32): re-used across the four batches
  constexpr uint32_t TM_AK = 0, TM_AV = 64, TM_KB = 128, TM_VB = 256, TM_T1K = 384, TM_T1V = 448;
  constexpr uint32_t TM_T2K = TM_AK, TM_T2V = TM_AV, TM_X = TM_KB, TM_Y = TM_VB, TM_GR = TM_T1K;
  constexpr int ET = 512;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sIn = base;                      // [2][k | v | dw | du | dk_in | A_w | A_u]
  unsigned char *sM0 = sIn + 2 * IN_BYTES;        // [64][128 B]: dA_w operand, then its first product
  unsigned char *sM1 = sM0 + T8;                  // [64][128 B]: dA_u operand, then its first product, then diag(beta) dA
  float *sBeta = reinterpret_cast<float *>(sM1 + T8);  // [2][64]
  float *sG = sBeta + 2 * C;                           // [2][64]
  // partial sums of the epilogue warps, one slot per (item parity, warp column group or lane quadrant, token): plain
  // stores, no atomics, every entry rewritten by exactly one lane per item; the scalar warp adds the four partials
  float *sDB = sG + 2 * C;                             // [2][4][64] dbeta rows per column group
  float *sDG = sDB + 8 * C;                            // [2][4][64] dg row sums per column group
  float *sDGC = sDG + 8 * C;                           // [2][4][64] dg column sums per lane quadrant
  __shared__ uint64_t full[2], empty[2], zero_done, b1_done, e1_done, b2_done, e2_done, b3_done, gr_done, e3_done, b4_done, acc_free, out_ready;
  __shared__ uint64_t scal_full[2], rows_done[2], ragged_sync;
  __shared__ int sRows[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const flab_args &a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int j = 0; j < 2; ++j) {
      mbar_init(&full[j], 1);
      mbar_init(&empty[j], 1);
    }
    mbar_init(&zero_done, 16);
    mbar_init(&b1_done, 1);
    mbar_init(&e1_done, 16);
    mbar_init(&b2_done, 1);
    mbar_init(&e2_done, 16);
    mbar_init(&b3_done, 1);
    mbar_init(&gr_done, 1);
    mbar_init(&e3_done, 16);
    mbar_init(&b4_done, 1);
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
  const bool has_dkin = a.x != nullptr;
  const int n_local = p.n_items > (int)blockIdx.x ? (p.n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  auto fail = [&](int code) {
    abort_flag = 1;
    atomicCAS(&tu_tc_error, 0, code);
  };
  // local item -> (sequence view, head, first token of the chunk inside the sequence, valid rows)
  auto locate = [&](int i, Seq &s, int &hd, int &t0, int &rows) {
    const int item = blockIdx.x + i * gridDim.x;
    hd = item % a.H;
    int n, it;
    chunk_of(a, item / a.H, n, it);
    s = seq_of(a, n);
    t0 = it * C;
    rows = min(C, s.len - t0);
  };

  if (warp == 16) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        const int b = i & 1, ph = (i >> 1) & 1;
        Seq s;
        int hd, t0, rows;
        locate(i, s, hd, t0, rows);
        const int tt = s.bos + t0, c1 = a.head_first ? tt : hd, c2 = a.head_first ? hd : tt;
        unsigned char *in = sIn + b * IN_BYTES;
        if (!mbar_wait(&empty[b], ph ^ 1)) { fail(81); break; }
        mbar_expect_tx(&full[b], IN_BYTES - (has_dkin ? 0 : T16) - (GATED ? 0 : T8));
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_4d(in + 0 * T16 + j * 8192, &m.k, &full[b], 64 * j, c1, c2, s.b);
          tma_load_4d(in + 1 * T16 + j * 8192, &m.v, &full[b], 64 * j, c1, c2, s.b);
          tma_load_4d(in + 2 * T16 + j * 8192, &m.dw, &full[b], 64 * j, c1, c2, s.b);
          tma_load_4d(in + 3 * T16 + j * 8192, &m.du, &full[b], 64 * j, c1, c2, s.b);
          if (has_dkin) tma_load_4d(in + 4 * T16 + j * 8192, &m.dkin, &full[b], 64 * j, c1, c2, s.b);
        }
        tma_load_4d(in + 5 * T16, &m.aw, &full[b], 0, c1, c2, s.b);
        if (GATED) tma_load_4d(in + 5 * T16 + T8, &m.au, &full[b], 0, c1, c2, s.b);
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t id_kk64 = instr_desc(64, 64, p.ab_fmt, 0, 0);    // x y^T      : A, B K-major
      const uint32_t id_mm64 = instr_desc(64, 64, p.ab_fmt, 1, 1);    // A^T T      : A, B MN-major
      const uint32_t id_mm128 = instr_desc(64, 128, p.ab_fmt, 1, 1);  // A^T dx, (beta dA)^T k
      const uint32_t id_km128 = instr_desc(64, 128, p.ab_fmt, 0, 1);  // dA k       : A K-major, B MN-major
      auto kx = [](int k) -> uint64_t { return (uint64_t)(((k >> 2) * 8192 + (k & 3) * 32) >> 4); };
      auto mx = [](int k) -> uint64_t { return (uint64_t)((k * 2048) >> 4); };
      const uint64_t dm0k = desc_kmajor(smem_u32(sM0), 0, 8192), dm1k = desc_kmajor(smem_u32(sM1), 0, 8192);
      const uint64_t dm0m = desc_mnmajor(smem_u32(sM0), 0, 8192), dm1m = desc_mnmajor(smem_u32(sM1), 0, 8192);
      int n_ragged = 0;
      // Only the row count of an item matters here (a ragged item waits for its zeroed rows). Its index arithmetic
      // (integer divisions) is done an item ahead, while this thread waits for the epilogue anyway: at the top of an
      // item it would delay the first batch, which the epilogue is waiting for.
      auto rows_of = [&](int i) -> int {
        if (i >= n_local) return C;
        Seq s;
        int hd, t0, rows;
        locate(i, s, hd, t0, rows);
        return rows;
      };
      int rows_next = rows_of(0);
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        const int b = i & 1, ph = (i >> 1) & 1, ip = i & 1;
        const int rows = rows_next;
        const uint32_t in = smem_u32(sIn + b * IN_BYTES);
        const uint32_t tk = in, tv = in + T16, tdw = in + 2 * T16, tdu = in + 3 * T16, taw = in + 5 * T16, tau = GATED ? taw + T8 : taw;
        const uint64_t dk_k = desc_kmajor(tk, 0, 8192), dv_k = desc_kmajor(tv, 0, 8192), dk_m = desc_mnmajor(tk, 0, 8192);
        const uint64_t ddw_k = desc_kmajor(tdw, 0, 8192), ddu_k = desc_kmajor(tdu, 0, 8192);
        const uint64_t ddw_m = desc_mnmajor(tdw, 0, 8192), ddu_m = desc_mnmajor(tdu, 0, 8192);
        const uint64_t daw_k = desc_kmajor(taw, 0, 8192), dau_k = desc_kmajor(tau, 0, 8192);
        const uint64_t daw_m = desc_mnmajor(taw, 0, 8192), dau_m = desc_mnmajor(tau, 0, 8192);
        if (!mbar_wait(&full[b], ph)) { fail(82); break; }
        if (rows < C) {  // the epilogue has zeroed the rows of dw, du past the end of the sequence
          if (!mbar_wait(&zero_done, n_ragged & 1)) { fail(83); break; }
          ++n_ragged;
        }
        if (i > 0 && !mbar_wait(&acc_free, ip ^ 1)) { fail(84); break; }
        fence_after_sync();
        // ---- B1
#pragma unroll
        for (int k = 0; k < 8; ++k) umma(tmem + TM_AK, ddw_k + kx(k), dk_k + kx(k), id_kk64, k > 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma(tmem + TM_AV, ddu_k + kx(k), dv_k + kx(k), id_kk64, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_KB, daw_m + mx(k), ddw_m + mx(k), id_mm128, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_VB, dau_m + mx(k), ddu_m + mx(k), id_mm128, k > 0);
        umma_commit(&b1_done);
        // ---- B2: (masked dA) A^T
        if (!mbar_wait(&e1_done, ip)) { fail(85); break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_T1K, dm0k + kx(k), daw_k + kx(k), id_kk64, k > 0);
        if (GATED) {
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem + TM_T1V, dm1k + kx(k), dau_k + kx(k), id_kk64, k > 0);
        }
        umma_commit(&b2_done);
        rows_next = rows_of(i + 1);
        // ---- B3: A^T (.)
        if (!mbar_wait(&e2_done, ip)) { fail(86); break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_T2K, daw_m + mx(k), dm0m + mx(k), id_mm64, k > 0);
        if (GATED) {
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem + TM_T2V, dau_m + mx(k), dm1m + mx(k), id_mm64, k > 0);
        }
        umma_commit(&b3_done);
        // k k^T (dbeta needs rowsum(dA * k k^T) = <(dA k)_i, k_i>, dg the same of dA_u) depends on nothing the epilogue
        // makes: it runs behind B3, in the columns the first product of the transform has left, and the epilogue turns
        // it into the dbeta / dg sums while B4 runs
#pragma unroll
        for (int k = 0; k < 8; ++k) umma(tmem + TM_GR, dk_k + kx(k), dk_k + kx(k), id_kk64, k > 0);
        umma_commit(&gr_done);
        // ---- B4: (diag(beta) dA) k + (diag(beta) dA)^T k in ONE accumulator (both are dk terms: beta_i (dA k)_i and
        //          ((beta dA)^T k)_i)
        if (!mbar_wait(&e3_done, ip)) { fail(87); break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_X, dm1k + kx(k), dk_m + mx(k), id_km128, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_X, dm1m + mx(k), dk_m + mx(k), id_mm128, 1);
        umma_commit(&b4_done);
      }
    }
  } else if (warp == 18) {
    // ------------------------------------------------------------------ output warp
    if (lane == 0) {
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        const int b = i & 1;
        Seq s;
        int hd, t0, rows;
        locate(i, s, hd, t0, rows);
        unsigned char *in = sIn + b * IN_BYTES;
        if (!mbar_wait(&out_ready, i & 1)) { fail(88); break; }
        if (rows == C) {  // (a ragged chunk was written out by the epilogue warps themselves)
          const int tt = s.bos + t0, c1 = a.head_first ? tt : hd, c2 = a.head_first ? hd : tt;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            tma_store_4d(&m.dk, in + 2 * T16 + j * 8192, 64 * j, c1, c2, s.b);
            tma_store_4d(&m.dv, in + 3 * T16 + j * 8192, 64 * j, c1, c2, s.b);
          }
          tma_store_commit();
          tma_store_wait_read();
        }
        mbar_arrive(&empty[b]);
      }
      tma_store_wait_all();
    }
  } else if (warp == 19) {
    // ------------------------------------------------------------------ scalar warp
    // Item i uses slot i & 1 of sBeta / sG / sDB / sDG / sRows.  Before a slot is handed to item i its previous user
    // (item i - 2) must be finished with it: the epilogue warps say so on rows_done, and their dbeta / dg rows are
    // written to global memory from here.
    float *dbeta_out = reinterpret_cast<float *>(a.dbeta), *dg_out = reinterpret_cast<float *>(a.dg);
    const float *dg_prev = reinterpret_cast<const float *>(a.dgk);  // dg of the preceding stage (optional): see flab_wy_bwd
    auto write_out = [&](int j) -> bool {
      const int slot = j & 1;
      if (!mbar_wait(&rows_done[slot], (j >> 1) & 1)) {
        fail(95);
        return false;
      }
      Seq s;
      int hd, t0, rows;
      locate(j, s, hd, t0, rows);
      const float *db = sDB + slot * 4 * C, *dgr = sDG + slot * 4 * C, *dgc = sDGC + slot * 4 * C;
      float x[2] = {0.f, 0.f};
      size_t o[2] = {0, 0};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = lane + 32 * h;
        if (t < rows) {
          o[h] = tok_off(a, s, hd, t0 + t, 1);
          dbeta_out[o[h]] = (db[t] + db[C + t]) + (db[2 * C + t] + db[3 * C + t]);
          if (GATED) {
            x[h] = ((dgr[t] + dgr[C + t]) + (dgr[2 * C + t] + dgr[3 * C + t])) - ((dgc[t] + dgc[C + t]) + (dgc[2 * C + t] + dgc[3 * C + t]));
            if (dg_prev) x[h] += dg_prev[o[h]];
          }
        }
      }
      if (GATED) {
        if (dg_prev) {
          // gradient w.r.t. the raw gate: suffix sums over the chunk's tokens (the reverse chunk-local cumsum the reference
          // applies at the end, fla/ops/gated_delta_rule/chunk.py:173-176); tokens lane + 32 first, then tokens lane
#pragma unroll
          for (int h = 1; h >= 0; --h) {
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
              const float y = __shfl_down_sync(0xffffffffu, x[h], off);
              if (lane + off < 32) x[h] += y;
            }
          }
          x[0] += __shfl_sync(0xffffffffu, x[1], 0);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
          if (lane + 32 * h < rows) dg_out[o[h]] = x[h];
      }
      return true;
    };
    // beta / gate of item i + 1 are fetched into registers before item i is published and before the wait for item i - 2:
    // the latency of these global loads is never exposed
    auto fetch = [&](int i, float (&bt)[2], float (&gt)[2], int &rows) {
      bt[0] = bt[1] = gt[0] = gt[1] = 0.f;
      rows = 0;
      if (i >= n_local) return;
      Seq s;
      int hd, t0;
      locate(i, s, hd, t0, rows);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = lane + 32 * h;
        if (t < rows) {
          const size_t o = tok_off(a, s, hd, t0 + t, 1);
          bt[h] = p.ab_fmt ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(a.beta)[o]) : __half2float(reinterpret_cast<const __half *>(a.beta)[o]);
          if (GATED) gt[h] = reinterpret_cast<const float *>(a.g)[o];
        }
      }
    };
    float cb[2], cg[2], nb[2], ng[2];
    int crows, nrows;
    fetch(0, cb, cg, crows);
    bool alive = true;
    for (int i = 0; i < n_local && alive && !abort_flag; ++i) {
      const int slot = i & 1;
      fetch(i + 1, nb, ng, nrows);
      if (i >= 2) alive = write_out(i - 2);
      __syncwarp();
      if (!alive) break;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sBeta[slot * C + lane + 32 * h] = cb[h];
        sG[slot * C + lane + 32 * h] = cg[h];
      }
      if (lane == 0) sRows[slot] = crows;
      __syncwarp();
      if (lane == 0) mbar_arrive(&scal_full[slot]);
#pragma unroll
      for (int h = 0; h < 2; ++h) cb[h] = nb[h], cg[h] = ng[h];
      crows = nrows;
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
    const int c128 = 32 * cq + 2 * t4;  // 128-column accumulators: columns c128 + 8 ni (+1), ni < 4
    const int c64 = 16 * cq + 2 * t4;   //  64-column accumulators: columns c64 + 8 ni (+1), ni < 2
    uint32_t o128_lo[4], o128_hi[4], o64_lo[2], o64_hi[2];  // byte offsets inside the swizzled tiles
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      const int col = c128 + 8 * ni;
      o128_lo[ni] = (uint32_t)(col >> 6) * 8192u + sw128_offset(row_lo, col & 63);
      o128_hi[ni] = (uint32_t)(col >> 6) * 8192u + sw128_offset(row_hi, col & 63);
    }
#pragma unroll
    for (int ni = 0; ni < 2; ++ni) {
      o64_lo[ni] = sw128_offset(row_lo, c64 + 8 * ni);
      o64_hi[ni] = sw128_offset(row_hi, c64 + 8 * ni);
    }
    auto ld2 = [&](const unsigned char *ptr) -> float2 {
      return p.ab_fmt ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(ptr))
                      : __half22float2(*reinterpret_cast<const __half2 *>(ptr));
    };
    auto st2 = [&](unsigned char *ptr, float x, float y) {
      if (p.ab_fmt) *reinterpret_cast<__nv_bfloat162 *>(ptr) = __floats2bfloat162_rn(x, y);
      else *reinterpret_cast<__half2 *>(ptr) = __floats2half2_rn(x, y);
    };
    auto rnd1 = [&](float x) -> float { return p.ab_fmt ? __bfloat162float(__float2bfloat16_rn(x)) : __half2float(__float2half_rn(x)); };
    int n_ragged = 0;
    for (int i = 0; i < n_local && !abort_flag; ++i) {
      const int b = i & 1, ph = (i >> 1) & 1, ip = i & 1;
      // beta, gate, row count and the zeroed dbeta / dg rows of this item, from the scalar warp
      if (!mbar_wait(&scal_full[ip], ph)) fail(96);
      const int rows = sRows[ip];
      unsigned char *in = sIn + b * IN_BYTES;
      unsigned char *tK = in, *tV = in + T16, *tDW = in + 2 * T16, *tDU = in + 3 * T16, *tDKI = in + 4 * T16;
      float *bs = sBeta + ip * C, *gs = sG + ip * C;
      float *dbs = sDB + (ip * 4 + cq) * C, *dgs = sDG + (ip * 4 + cq) * C, *dgc = sDGC + (ip * 4 + wq) * C;
      const float b_lo = bs[row_lo], b_hi = bs[row_hi], g_lo = gs[row_lo], g_hi = gs[row_hi];
      // decay e^{g_i - g_j} of this thread's eight entries of the 64x64 blocks (strict lower triangle), computed here,
      // ahead of the first wait, so that E3, which sits on the chain between two products, only multiplies
      float dec[2][4];
      if (GATED) {
#pragma unroll
        for (int ni = 0; ni < 2; ++ni)
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int row = (r >> 1) ? row_hi : row_lo, cc = c64 + 8 * ni + (r & 1);
            dec[ni][r] = row > cc ? __expf(fminf(((r >> 1) ? g_hi : g_lo) - gs[cc], 0.f)) : 0.f;
          }
      }
      if (!mbar_wait(&full[b], ph)) fail(89);
      if (rows < C) {
        // ragged last chunk: the rows of dw, du past the end of the sequence hold another sequence's data
        for (int e = tid; e < (C - rows) * 32; e += ET) {
          const int r_ = rows + (e >> 5), pc = e & 31;  // 32 16-byte pieces per row: 16 of dw, 16 of du
          unsigned char *t = (pc & 16) ? tDU : tDW;
          *reinterpret_cast<int4 *>(t + ((pc & 15) >> 3) * 8192 + r_ * 128 + ((pc & 7) << 4)) = make_int4(0, 0, 0, 0);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&zero_done);
      }
      // ---- E1: masked dA operands; then dv, first part of dk and dbeta while the tensor core transforms dA
      if (!mbar_wait(&b1_done, ip)) fail(90);
      fence_after_sync();
      {
        float ak[2][4], av[2][4];
        tmem_ld_frag<2>(tmem + lane_base + TM_AK + 16 * cq, ak);
        tmem_ld_frag<2>(tmem + lane_base + TM_AV + 16 * cq, av);
        tmem_ld_wait();
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
          const int col = c64 + 8 * ni;
          const float bc0 = bs[col], bc1 = bs[col + 1];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int row = hf ? row_hi : row_lo;
            const bool m0_ = row > col && row < rows, m1_ = row > col + 1 && row < rows;
            const uint32_t off = hf ? o64_hi[ni] : o64_lo[ni];
            if (GATED) {
              st2(sM0 + off, m0_ ? ak[ni][2 * hf] * bc0 : 0.f, m1_ ? ak[ni][2 * hf + 1] * bc1 : 0.f);
              st2(sM1 + off, m0_ ? av[ni][2 * hf] * bc0 : 0.f, m1_ ? av[ni][2 * hf + 1] * bc1 : 0.f);
            } else {
              st2(sM0 + off, m0_ ? (ak[ni][2 * hf] + av[ni][2 * hf]) * bc0 : 0.f,
                  m1_ ? (ak[ni][2 * hf + 1] + av[ni][2 * hf + 1]) * bc1 : 0.f);
            }
          }
        }
      }
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&e1_done);
      // dv and its part of dbeta, while the tensor core runs the first product of the transform
      float db_lo = 0.f, db_hi = 0.f;
      {
        float vb[4][4];
        tmem_ld_frag<4>(tmem + lane_base + TM_VB + 32 * cq, vb);
        tmem_ld_wait();
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
          const float2 v_lo = ld2(tV + o128_lo[ni]), v_hi = ld2(tV + o128_hi[ni]);
          db_lo += vb[ni][0] * v_lo.x + vb[ni][1] * v_lo.y;
          db_hi += vb[ni][2] * v_hi.x + vb[ni][3] * v_hi.y;
          st2(tDU + o128_lo[ni], vb[ni][0] * b_lo, vb[ni][1] * b_lo);  // dv, over du (the tensor core is done with it)
          st2(tDU + o128_hi[ni], vb[ni][2] * b_hi, vb[ni][3] * b_hi);
        }
      }
      // ---- E2: first product of the transform, rounded, becomes the operand of the second
      if (!mbar_wait(&b2_done, ip)) fail(91);
      fence_after_sync();
      {
        float t1k[2][4], t1v[2][4];
        tmem_ld_frag<2>(tmem + lane_base + TM_T1K + 16 * cq, t1k);
        if (GATED) tmem_ld_frag<2>(tmem + lane_base + TM_T1V + 16 * cq, t1v);
        tmem_ld_wait();
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
          st2(sM0 + o64_lo[ni], t1k[ni][0], t1k[ni][1]);
          st2(sM0 + o64_hi[ni], t1k[ni][2], t1k[ni][3]);
          if (GATED) {
            st2(sM1 + o64_lo[ni], t1v[ni][0], t1v[ni][1]);
            st2(sM1 + o64_hi[ni], t1v[ni][2], t1v[ni][3]);
          }
        }
      }
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&e2_done);
      // the first part of dk and of dbeta, while the tensor core runs the second product of the transform
      float dk1[4][4];
      {
        tmem_ld_frag<4>(tmem + lane_base + TM_KB + 32 * cq, dk1);
        tmem_ld_wait();
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
          const float2 k_lo = ld2(tK + o128_lo[ni]), k_hi = ld2(tK + o128_hi[ni]);
          db_lo += dk1[ni][0] * k_lo.x + dk1[ni][1] * k_lo.y;
          db_hi += dk1[ni][2] * k_hi.x + dk1[ni][3] * k_hi.y;
          dk1[ni][0] *= b_lo, dk1[ni][1] *= b_lo, dk1[ni][2] *= b_hi, dk1[ni][3] *= b_hi;
        }
      }
      // ---- E3: dA = -strict_lower(.) (+ decayed dA_u), and diag(beta) dA
      if (!mbar_wait(&b3_done, ip)) fail(92);
      fence_after_sync();
      float dA2[2][4];  // decayed dA_u (gated), for dg
      float dAt[2][4];  // dA, for dbeta
      {
        float t2k[2][4], t2v[2][4];
        tmem_ld_frag<2>(tmem + lane_base + TM_T2K + 16 * cq, t2k);
        if (GATED) tmem_ld_frag<2>(tmem + lane_base + TM_T2V + 16 * cq, t2v);
        tmem_ld_wait();
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
          const int col = c64 + 8 * ni;
          float d[4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int row = (r >> 1) ? row_hi : row_lo, cc = col + (r & 1);
            float x = row > cc ? rnd1(-t2k[ni][r]) : 0.f;
            if (GATED) {
              const float x2 = rnd1(-t2v[ni][r]) * dec[ni][r];
              dA2[ni][r] = x2;
              x = rnd1(x + x2);
            }
            d[r] = x;
            dAt[ni][r] = x;
          }
          st2(sM1 + o64_lo[ni], d[0] * b_lo, d[1] * b_lo);
          st2(sM1 + o64_hi[ni], d[2] * b_hi, d[3] * b_hi);
        }
      }
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&e3_done);
      // ---- the dbeta / dg sums that need k k^T, while the tensor core runs B4
      if (!mbar_wait(&gr_done, ip)) fail(98);
      fence_after_sync();
      {
        float gr[2][4];
        tmem_ld_frag<2>(tmem + lane_base + TM_GR + 16 * cq, gr);
        tmem_ld_wait();
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {  // <(dA k)_i, k_i> = sum_j dA_ij (k k^T)_ij
          db_lo += dAt[ni][0] * gr[ni][0] + dAt[ni][1] * gr[ni][1];
          db_hi += dAt[ni][2] * gr[ni][2] + dAt[ni][3] * gr[ni][3];
        }
        if (GATED) {
          float r_lo = 0.f, r_hi = 0.f;
#pragma unroll
          for (int ni = 0; ni < 2; ++ni) {
            const float p0 = dA2[ni][0] * gr[ni][0] * b_lo, p1 = dA2[ni][1] * gr[ni][1] * b_lo;
            const float p2 = dA2[ni][2] * gr[ni][2] * b_hi, p3 = dA2[ni][3] * gr[ni][3] * b_hi;
            r_lo += p0 + p1;
            r_hi += p2 + p3;
            float c0 = p0 + p2, c1 = p1 + p3;
            c0 += __shfl_xor_sync(0xffffffffu, c0, 4);
            c0 += __shfl_xor_sync(0xffffffffu, c0, 8);
            c0 += __shfl_xor_sync(0xffffffffu, c0, 16);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 4);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 8);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 16);
            if (g8 == 0) {
              dgc[c64 + 8 * ni] = c0;
              dgc[c64 + 8 * ni + 1] = c1;
            }
          }
          r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 1);
          r_lo += __shfl_xor_sync(0xffffffffu, r_lo, 2);
          r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 1);
          r_hi += __shfl_xor_sync(0xffffffffu, r_hi, 2);
          if (t4 == 0) {
            dgs[row_lo] = r_lo;
            dgs[row_hi] = r_hi;
          }
        }
      }
      // ---- E4: dk, dbeta
      if (!mbar_wait(&b4_done, ip)) fail(93);
      fence_after_sync();
      {
        float xy[4][4];
        tmem_ld_frag<4>(tmem + lane_base + TM_X + 32 * cq, xy);
        tmem_ld_wait();
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_free);
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
          float o0 = dk1[ni][0] + xy[ni][0], o1 = dk1[ni][1] + xy[ni][1];
          float o2 = dk1[ni][2] + xy[ni][2], o3 = dk1[ni][3] + xy[ni][3];
          if (has_dkin) {
            const float2 i_lo = ld2(tDKI + o128_lo[ni]), i_hi = ld2(tDKI + o128_hi[ni]);
            o0 += i_lo.x, o1 += i_lo.y, o2 += i_hi.x, o3 += i_hi.y;
          }
          st2(tDW + o128_lo[ni], o0, o1);  // dk, over dw
          st2(tDW + o128_hi[ni], o2, o3);
        }
        db_lo += __shfl_xor_sync(0xffffffffu, db_lo, 1);
        db_lo += __shfl_xor_sync(0xffffffffu, db_lo, 2);
        db_hi += __shfl_xor_sync(0xffffffffu, db_hi, 1);
        db_hi += __shfl_xor_sync(0xffffffffu, db_hi, 2);
        if (t4 == 0) {
          dbs[row_lo] = db_lo;
          dbs[row_hi] = db_hi;
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&rows_done[ip]);  // this warp's share of the dbeta / dg rows is in shared memory
      if (rows < C) {
        // ragged last chunk of a sequence: a tile store would write past its end, so the epilogue warps copy the valid
        // rows themselves once every warp has finished its part of the dk / dv tiles
        if (lane == 0) mbar_arrive(&ragged_sync);
        if (!mbar_wait(&ragged_sync, n_ragged & 1)) fail(97);
        ++n_ragged;
        Seq s;
        int hd, t0, rows_;
        locate(i, s, hd, t0, rows_);
        const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V);
        const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V);
        for (int e = tid; e < rows * 16; e += ET) {
          const int r_ = e >> 4, c_ = (e & 15) * 8;
          const uint32_t so = (uint32_t)(c_ >> 6) * 8192u + sw128_offset(r_, c_ & 63);
          *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.dk) + offk + (size_t)r_ * ks + c_) = *reinterpret_cast<const int4 *>(tDW + so);
          *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.dv) + offv + (size_t)r_ * vs + c_) = *reinterpret_cast<const int4 *>(tDU + so);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&out_ready);  // this warp is done with the item's tiles
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <bool GATED> static int launch_tc_wy_bwd(const flab_args *a, cudaStream_t stream) {
  TcWyMaps m;
  if (int e = make_token_map(&m.k, a->k, a, a->K)) return e;
  if (int e = make_token_map(&m.v, a->v, a, a->V)) return e;
  if (int e = make_token_map(&m.dw, a->dw, a, a->K)) return e;
  if (int e = make_token_map(&m.du, a->du, a, a->V)) return e;
  if (int e = make_token_map(&m.dkin, a->x ? a->x : a->k, a, a->K)) return e;
  if (int e = make_token_map(&m.aw, a->aw, a, C)) return e;
  if (int e = make_token_map(&m.au, GATED ? a->au : a->aw, a, C)) return e;
  if (int e = make_token_map(&m.dk, a->dk, a, a->K)) return e;
  if (int e = make_token_map(&m.dv, a->dv, a, a->V)) return e;
  TcWyParams p;
  p.a = *a;
  p.n_items = a->NT * a->H;
  p.ab_fmt = a->dtype == FLAB_BF16 ? 1 : 0;
  const size_t smem = 1024 + 2 * (size_t)(5 * 16384 + 2 * 8192) + 2 * 8192 + 28 * C * sizeof(float);
  auto kern = tc_wy_bwd_kernel<GATED>;
  if (int e = set_smem(kern, smem)) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.n_items < sms ? p.n_items : sms;
  kern<<<grid, 640, smem, stream>>>(m, p);
  return check_launch("wy_bwd(tc)");
}

// Returns 1 if the tcgen05 kernel took the call, 0 if the shape is outside its domain, < 0 on error.
int tc_wy_bwd_try(const flab_args *a, cudaStream_t stream) {
  if (a->dtype != FLAB_BF16 && a->dtype != FLAB_FP16) return 0;
  if (a->K != 128 || a->V != 128) return 0;
  const void *ptrs[9] = {a->k, a->v, a->dw, a->du, a->x, a->aw, a->au, a->dk, a->dv};
  for (int i = 0; i < 9; ++i)
    if (ptrs[i] && reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return 0;
  const int rc = a->g ? launch_tc_wy_bwd<true>(a, stream) : launch_tc_wy_bwd<false>(a, stream);
  return rc < 0 ? rc : 1;
}

}  // namespace flab
