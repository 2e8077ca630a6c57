// tcgen05 / TMA version of the forward WY / UT transform (bf16 / fp16, K = V = 128):
//   A_w = (I + tril(diag(beta) k k^T, -1))^-1,  A_u = D A_w D^-1 (D = diag(e^b); gated only),
//   w = A_w (beta k),  u = A_u (beta v)
//   (fla/ops/delta_rule/wy_fast.py:94-253, 436-530; fla/ops/gated_delta_rule/wy_fast.py:111-317)
// Persistent kernel, one CTA per SM, work item = (chunk, head).  Twenty warps:
//   warps 0-7 / 8-15 : two epilogue groups working on even / odd items.  The 64x64 fp32 inverse is SIMT work
//                      (forward substitution + fp32 block merges, wy_inverse.cuh) with little parallelism, so one
//                      group inverts while the other group's products, conversions and stores run.
//   warp 16 : TMA producer - k and v of an item into a ring of three stages shared by the groups, so that the
//             next item of a group is already resident while the previous one is still being stored
//   warp 17 : MMA issuer   - k k^T, then (A_w diag(beta)) k and (A_u diag(beta)) v, software-pipelined over
//                            the two groups; each group owns 256 TMEM columns (the Gram block is re-used by w)
//   warps 18, 19 : output  - tile stores of A_w, A_u (after the inverse) and of w, u (which the epilogue builds over
//                            the k and v tiles), one warp per group; then the buffer goes back to the producer
// beta enters the Gram matrix as a row factor of the fp32 product and w, u as a column factor of A, so no
// beta-scaled copy of k or v exists.  All waits are bounded; a timeout records an id in the unit's error word
// and a group leaves as one at its next barrier.
#include "tc.cuh"
#include "wy_inverse.cuh"

FLAB_TC_DEFINE_ERROR_WORD(tc_wy_fwd_error)

namespace flab {

struct TcWfParams {
  flab_args a;
  int n_items;  // NT * H
  int ab_fmt;   // 1 bf16, 0 fp16
};

struct TcWfMaps {
  CUtensorMap k, v, aw, au, w, u;
};

template <bool GATED>
__global__ void __launch_bounds__(640, 1) tc_wy_fwd_kernel(const __grid_constant__ TcWfMaps m, const TcWfParams p) {
  using namespace tc;
  constexpr uint32_t T16 = 16384, T8 = 8192;
  constexpr uint32_t F_BYTES = C * LDL * 4 + 32 * 33 * 4;  // fp32 work matrix + scratch of the inverse
  constexpr uint32_t F_PAD = (F_BYTES + 1023) & ~1023u;
  constexpr int NS = 3;                                    // k / v stages
  constexpr uint32_t S_BYTES = 2 * T16;                    // one stage: k | v (replaced in place by w | u)
  constexpr uint32_t G_BYTES = 4 * T8 + F_PAD;             // one group's private buffers
  constexpr uint32_t TM_GROUP = 256, TM_W = 0, TM_U = 128;  // per group; the Gram block sits in the first 64 columns of w

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float *sScal = reinterpret_cast<float *>(base + NS * S_BYTES + 2 * G_BYTES);  // [2 groups][beta 64 | gate 64]
  __shared__ uint64_t full[NS], empty[NS], g1_done[2], e1_done[2], g23_done[2], acc_free[2], out_ready[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;
  __shared__ volatile int abort_snap[2][2];

  const flab_args &a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int j = 0; j < NS; ++j) {
      mbar_init(&full[j], 1);
      mbar_init(&empty[j], 1);
    }
    for (int j = 0; j < 2; ++j) {
      mbar_init(&g1_done[j], 1);
      mbar_init(&e1_done[j], 8);
      mbar_init(&g23_done[j], 1);
      mbar_init(&acc_free[j], 8);
      mbar_init(&out_ready[j], 8);
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
  const int n_local = p.n_items > (int)blockIdx.x ? (p.n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  auto fail = [&](int code) {
    abort_flag = 1;
    atomicCAS(&tu_tc_error, 0, code);
  };
  auto locate = [&](int i, Seq &s, int &hd, int &t0, int &rows) {
    const int item = blockIdx.x + i * gridDim.x;
    hd = item % a.H;
    int n, it;
    chunk_of(a, item / a.H, n, it);
    s = seq_of(a, n);
    t0 = it * C;
    rows = min(C, s.len - t0);
  };
  // stage: k | v; group buffers: A_w | A_u | A_w diag(beta) | A_u diag(beta) | fp32 work
  auto sbuf = [&](int st) -> unsigned char * { return base + st * S_BYTES; };
  auto gbuf = [&](int g) -> unsigned char * { return base + NS * S_BYTES + g * G_BYTES; };

  if (warp == 16) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < n_local && !abort_flag; ++i) {
        const int st = i % NS, sph = (i / NS) & 1;
        Seq s;
        int hd, t0, rows;
        locate(i, s, hd, t0, rows);
        const int tt = s.bos + t0, c1 = a.head_first ? tt : hd, c2 = a.head_first ? hd : tt;
        if (!mbar_wait(&empty[st], sph ^ 1)) { fail(101); break; }
        mbar_expect_tx(&full[st], S_BYTES);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_4d(sbuf(st) + j * 8192, &m.k, &full[st], 64 * j, c1, c2, s.b);
          tma_load_4d(sbuf(st) + T16 + j * 8192, &m.v, &full[st], 64 * j, c1, c2, s.b);
        }
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t id_g = instr_desc(64, 64, p.ab_fmt, 0, 0);    // k k^T       : A, B K-major
      const uint32_t id_w = instr_desc(64, 128, p.ab_fmt, 0, 1);   // (A beta) x  : A K-major, B MN-major
      auto kx = [](int k) -> uint64_t { return (uint64_t)(((k >> 2) * 8192 + (k & 3) * 32) >> 4); };
      auto mx = [](int k) -> uint64_t { return (uint64_t)((k * 2048) >> 4); };
      auto gram = [&](int i) -> bool {
        const int g = i & 1, ph = (i >> 1) & 1, st = i % NS, sph = (i / NS) & 1;
        if (!mbar_wait(&full[st], sph)) { fail(102); return false; }
        if (i >= 2 && !mbar_wait(&acc_free[g], ph ^ 1)) { fail(103); return false; }  // w of the group's previous item has been read
        fence_after_sync();
        const uint64_t dk = desc_kmajor(smem_u32(sbuf(st)), 0, 8192);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma(tmem + g * TM_GROUP + TM_W, dk + kx(k), dk + kx(k), id_g, k > 0);
        umma_commit(&g1_done[g]);
        return true;
      };
      bool ok = n_local > 0 ? gram(0) : true;
      for (int i = 0; i < n_local && ok && !abort_flag; ++i) {
        const int g = i & 1, ph = (i >> 1) & 1;
        if (i + 1 < n_local) ok = gram(i + 1);  // the other group's Gram matrix before this group's products
        if (!ok) break;
        if (!mbar_wait(&e1_done[g], ph)) { fail(104); break; }
        fence_after_sync();
        const uint32_t gb = smem_u32(gbuf(g)), sb = smem_u32(sbuf(i % NS));
        const uint64_t dkm = desc_mnmajor(sb, 0, 8192), dvm = desc_mnmajor(sb + T16, 0, 8192);
        const uint64_t dabw = desc_kmajor(gb + 2 * T8, 0, 8192), dabu = desc_kmajor(gb + (GATED ? 3 : 2) * T8, 0, 8192);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + g * TM_GROUP + TM_W, dabw + kx(k), dkm + mx(k), id_w, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + g * TM_GROUP + TM_U, dabu + kx(k), dvm + mx(k), id_w, k > 0);
        umma_commit(&g23_done[g]);
      }
    }
  } else if (warp >= 18) {
    // ------------------------------------------------------------------ output warps (one per group)
    if (lane == 0) {
      const int g = warp - 18;
      for (int i = g; i < n_local && !abort_flag; i += 2) {
        const int ph = (i >> 1) & 1;
        Seq s;
        int hd, t0, rows;
        locate(i, s, hd, t0, rows);
        const int tt = s.bos + t0, c1 = a.head_first ? tt : hd, c2 = a.head_first ? hd : tt;
        unsigned char *gb = gbuf(g), *sb = sbuf(i % NS);
        if (!mbar_wait(&e1_done[g], ph)) { fail(105); break; }
        if (rows == C) {  // (a ragged chunk is written out by the epilogue warps themselves)
          tma_store_4d(&m.aw, gb, 0, c1, c2, s.b);
          if (GATED) tma_store_4d(&m.au, gb + T8, 0, c1, c2, s.b);
          tma_store_commit();
        }
        if (!mbar_wait(&out_ready[g], ph)) { fail(106); break; }
        if (rows == C) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            tma_store_4d(&m.w, sb + j * 8192, 64 * j, c1, c2, s.b);
            tma_store_4d(&m.u, sb + T16 + j * 8192, 64 * j, c1, c2, s.b);
          }
          tma_store_commit();
          tma_store_wait_read();
        }
        mbar_arrive(&empty[i % NS]);
      }
      tma_store_wait_all();
    }
  } else {
    // ------------------------------------------------------------------ epilogue groups (warps 0-7, 8-15)
    const int g = warp >> 3, gw = warp & 7, gtid = tid & 255;
    const int wq = gw & 3, ch = gw >> 2, g8 = lane >> 2, t4 = lane & 3;
    const uint32_t tm = tmem + g * TM_GROUP + ((uint32_t)(32 * wq) << 16);
    const int row_lo = 16 * wq + g8, row_hi = row_lo + 8;
    unsigned char *gb = gbuf(g);
    unsigned char *sAw = gb, *sAu = sAw + T8, *sAbw = sAu + T8, *sAbu = sAbw + T8;
    float *sF = reinterpret_cast<float *>(sAbu + T8), *sScr = sF + C * LDL;
    float *bs = sScal + g * 2 * C, *gs = bs + C;
    auto grp_sync = [&]() { asm volatile("bar.sync %0, 256;" ::"r"(1 + g) : "memory"); };
    auto pack8 = [&](const float *x) -> int4 {
      int4 r;
      if (p.ab_fmt) {
        __nv_bfloat162 *q = reinterpret_cast<__nv_bfloat162 *>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
      } else {
        __half2 *q = reinterpret_cast<__half2 *>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = __floats2half2_rn(x[2 * j], x[2 * j + 1]);
      }
      return r;
    };
    auto unpack8 = [&](const int4 &r, float *x) {
      if (p.ab_fmt) {
        const __nv_bfloat162 *q = reinterpret_cast<const __nv_bfloat162 *>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(q[j]);
          x[2 * j] = f.x, x[2 * j + 1] = f.y;
        }
      } else {
        const __half2 *q = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(q[j]);
          x[2 * j] = f.x, x[2 * j + 1] = f.y;
        }
      }
    };
    auto st2 = [&](unsigned char *ptr, float x, float y) {
      if (p.ab_fmt) *reinterpret_cast<__nv_bfloat162 *>(ptr) = __floats2bfloat162_rn(x, y);
      else *reinterpret_cast<__half2 *>(ptr) = __floats2half2_rn(x, y);
    };
    // Where the group's next item lies, and beta and gate of its token `gtid`: worked out one of the group's items ahead,
    // while the tensor core runs the current item's products, so that neither the index arithmetic (integer divisions)
    // nor the global loads sit on the group's chain
    Seq s_n;
    int hd_n = 0, t0_n = 0, rows_n = 0;
    float b_pf = 0.f, g_pf = 0.f;
    auto fetch = [&](int i) {
      b_pf = 0.f, g_pf = 0.f, rows_n = 0;
      if (i >= n_local) return;
      locate(i, s_n, hd_n, t0_n, rows_n);
      if (gtid < rows_n) {  // (rows_n <= 64)
        const size_t o = tok_off(a, s_n, hd_n, t0_n + gtid, 1);
        b_pf = p.ab_fmt ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(a.beta)[o]) : __half2float(reinterpret_cast<const __half *>(a.beta)[o]);
        if (GATED) g_pf = reinterpret_cast<const float *>(a.g)[o];
      }
    };
    fetch(g);
    for (int i = g; i < n_local; i += 2) {
      const int ph = (i >> 1) & 1;
      unsigned char *tK = sbuf(i % NS), *tV = tK + T16;
      const Seq s = s_n;
      const int hd = hd_n, t0 = t0_n, rows = rows_n;
      if (gtid < C) {
        bs[gtid] = b_pf;
        gs[gtid] = g_pf;
      }
      if (gtid == 0) abort_snap[g][ph] = abort_flag;
      grp_sync();
      if (abort_snap[g][ph]) break;
      // ---- E1: Gram block -> fp32 work matrix -> inverse -> A (stored), A diag(beta) (operands)
      if (!mbar_wait(&g1_done[g], ph)) fail(107);
      fence_after_sync();
      {
        float gr[4][4];
        tmem_ld_frag<4>(tm + TM_W + 32 * ch, gr);
        tmem_ld_wait();
        const float b_lo = bs[row_lo], b_hi = bs[row_hi];
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int row = (r >> 1) ? row_hi : row_lo, col = 32 * ch + 8 * ni + 2 * t4 + (r & 1);
            sF[row * LDL + col] = (row > col && row < rows) ? -gr[ni][r] * ((r >> 1) ? b_hi : b_lo) : 0.f;
          }
      }
      fence_before_sync();
      grp_sync();
      if (g == 0) tri_inverse8<1, 1>(sF, sScr, gtid);
      else tri_inverse8<1, 2>(sF, sScr, gtid);
      for (int e = gtid; e < C * 8; e += 256) {
        const int r_ = e >> 3, c_ = (e & 7) * 8;
        const uint32_t off = (uint32_t)r_ * 128u + ((uint32_t)((c_ >> 3) ^ (r_ & 7)) << 4);
        const float *src = sF + r_ * LDL + c_;
        float x[8], y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = src[j];
        int4 pk = pack8(x);
        *reinterpret_cast<int4 *>(sAw + off) = pk;
        unpack8(pk, y);  // the column factor is applied to the ROUNDED A, as the recompute entry does from the stored A
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] *= bs[c_ + j];
        *reinterpret_cast<int4 *>(sAbw + off) = pack8(y);
        if (GATED) {
          const float gr_ = gs[r_];
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] *= __expf(fminf(gr_ - gs[c_ + j], 0.f));
          pk = pack8(x);
          *reinterpret_cast<int4 *>(sAu + off) = pk;
          unpack8(pk, y);
#pragma unroll
          for (int j = 0; j < 8; ++j) y[j] *= bs[c_ + j];
          *reinterpret_cast<int4 *>(sAbu + off) = pack8(y);
        }
      }
      fence_proxy_async();
      if (rows < C) {
        // ragged last chunk: the valid rows of A go out with ordinary stores
        grp_sync();
        const size_t as_ = tok_stride(a, C), offa = tok_off(a, s, hd, t0, C);
        for (int e = gtid; e < rows * 8; e += 256) {
          const int r_ = e >> 3, c_ = (e & 7) * 8;
          const uint32_t off = (uint32_t)r_ * 128u + ((uint32_t)((c_ >> 3) ^ (r_ & 7)) << 4);
          *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.aw) + offa + (size_t)r_ * as_ + c_) = *reinterpret_cast<const int4 *>(sAw + off);
          if (GATED) *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.au) + offa + (size_t)r_ * as_ + c_) = *reinterpret_cast<const int4 *>(sAu + off);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&e1_done[g]);
      fetch(i + 2);
      // ---- E2: w, u -> rounded, over the k and v tiles
      if (!mbar_wait(&g23_done[g], ph)) fail(108);
      fence_after_sync();
      {
        float wv[8][4], uv[8][4];
        tmem_ld_frag<8>(tm + TM_W + 64 * ch, wv);
        tmem_ld_frag<8>(tm + TM_U + 64 * ch, uv);
        tmem_ld_wait();
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_free[g]);
#pragma unroll
        for (int ni = 0; ni < 8; ++ni) {
          const int col = 8 * ni + 2 * t4;  // inside the 64-column box `ch`
          const uint32_t o_lo = (uint32_t)ch * 8192u + sw128_offset(row_lo, col), o_hi = (uint32_t)ch * 8192u + sw128_offset(row_hi, col);
          st2(tK + o_lo, wv[ni][0], wv[ni][1]);
          st2(tK + o_hi, wv[ni][2], wv[ni][3]);
          st2(tV + o_lo, uv[ni][0], uv[ni][1]);
          st2(tV + o_hi, uv[ni][2], uv[ni][3]);
        }
      }
      fence_proxy_async();
      if (rows < C) {
        grp_sync();
        const size_t ks = tok_stride(a, a.K), vs = tok_stride(a, a.V);
        const size_t offk = tok_off(a, s, hd, t0, a.K), offv = tok_off(a, s, hd, t0, a.V);
        for (int e = gtid; e < rows * 16; e += 256) {
          const int r_ = e >> 4, c_ = (e & 15) * 8;
          const uint32_t so = (uint32_t)(c_ >> 6) * 8192u + sw128_offset(r_, c_ & 63);
          *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.w) + offk + (size_t)r_ * ks + c_) = *reinterpret_cast<const int4 *>(tK + so);
          *reinterpret_cast<int4 *>(reinterpret_cast<bf16 *>(a.u) + offv + (size_t)r_ * vs + c_) = *reinterpret_cast<const int4 *>(tV + so);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&out_ready[g]);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <bool GATED> static int launch_tc_wy_fwd(const flab_args *a, cudaStream_t stream) {
  TcWfMaps m;
  if (int e = make_token_map(&m.k, a->k, a, a->K)) return e;
  if (int e = make_token_map(&m.v, a->v, a, a->V)) return e;
  if (int e = make_token_map(&m.aw, a->aw, a, C)) return e;
  if (int e = make_token_map(&m.au, GATED ? a->au : a->aw, a, C)) return e;
  if (int e = make_token_map(&m.w, a->w, a, a->K)) return e;
  if (int e = make_token_map(&m.u, a->u, a, a->V)) return e;
  TcWfParams p;
  p.a = *a;
  p.n_items = a->NT * a->H;
  p.ab_fmt = a->dtype == FLAB_BF16 ? 1 : 0;
  constexpr uint32_t F_PAD = ((C * LDL * 4 + 32 * 33 * 4) + 1023) & ~1023u;
  const size_t smem = 1024 + 3 * (size_t)(2 * 16384) + 2 * (size_t)(4 * 8192 + F_PAD) + 4 * C * sizeof(float);
  auto kern = tc_wy_fwd_kernel<GATED>;
  if (int e = set_smem(kern, smem)) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = p.n_items < sms ? p.n_items : sms;
  kern<<<grid, 640, smem, stream>>>(m, p);
  return check_launch("wy_fwd(tc)");
}

// Returns 1 if the tcgen05 kernel took the call, 0 if the shape is outside its domain, < 0 on error.
int tc_wy_fwd_try(const flab_args *a, cudaStream_t stream) {
  if (a->dtype != FLAB_BF16 && a->dtype != FLAB_FP16) return 0;
  if (a->K != 128 || a->V != 128) return 0;
  const void *ptrs[6] = {a->k, a->v, a->aw, a->au, a->w, a->u};
  for (int i = 0; i < 6; ++i)
    if (ptrs[i] && reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return 0;
  const int rc = a->g ? launch_tc_wy_fwd<true>(a, stream) : launch_tc_wy_fwd<false>(a, stream);
  return rc < 0 ? rc : 1;
}

}  // namespace flab
