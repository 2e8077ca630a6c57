// tcgen05 / TMA version of the forward delta-rule state scan (bf16 / fp16, K = 128, V % 64 == 0):
//   per chunk t:  h[t] = S;  v_new = u - e^{b} (w S);  S <- e^{b_L} S + k^T (e^{b_L - b} v_new)
//   (fla/ops/common/chunk_delta_h.py:248-321)
// One CTA per (sequence, head, value tile of 128 or 64 columns); the chunks of a sequence form a serial
// chain, so the kernel is organised around the latency of one step:
//   warp EW     : TMA producer - streams the w, k, u tiles of the next chunks into a ring of stages
//   warp EW + 1 : MMA issuer   - P = w S (M = 64 tokens) and dS = k^T op (M = 128 state rows) into TMEM
//   warps 0 .. EW-1 (EW = 16 for a 128-column tile): epilogue - hold the fp32 state in REGISTERS (thread =
//                 one state row x 32 columns), so the tensor core only ever produces the increment dS:
//                 phase A: S <- e^{b_L} S + dS; round, write as the swizzled B operand of the next
//                          product and, straight from registers, to h[t] (128 contiguous bytes per thread)
//                 phase B: P -> v_new (staged, coalesced store) and op = e^{b_L-b} v_new (swizzled operand)
// A step is phase A -> MMA -> phase B -> MMA; nothing else sits on the chain (tile loads run stages ahead,
// the gates of the next chunk are fetched into a register a chunk early, stores are issued after the arrive
// that releases the tensor core).  All waits are bounded; a timeout records an id in the unit's error word,
// and the epilogue warps leave together at their next common barrier.
#include "tc.cuh"

FLAB_TC_DEFINE_ERROR_WORD(tc_delta_h_error)

namespace flab {

struct TcDhParams {
  flab_args a;
  int v_tiles;  // V / BV
  int ab_fmt;   // 1 bf16, 0 fp16
};

template <int VB /* BV / 64 */, int NS>
__global__ void __launch_bounds__(64 * (4 * VB + 1), 1)
tc_delta_fwd_h_kernel(const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapU, const __grid_constant__ CUtensorMap mapH,
                      const __grid_constant__ CUtensorMap mapVn, const TcDhParams p) {
  using namespace tc;
  constexpr int K = 128, BV = 64 * VB, NC = 32;  // NC: state columns per epilogue thread
  constexpr int EW = BV / 8, ET = 32 * EW;         // epilogue warps (4 lane quadrants x BV/32 column groups), threads
  constexpr uint32_t KT_BYTES = 2 * 8192, U_BYTES = VB * 8192, STAGE_BYTES = 2 * KT_BYTES + U_BYTES;
  constexpr uint32_t TM_DS = 0, TM_P = 128;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sStage = base;                        // [NS][w | k | u]
  unsigned char *sS = sStage + NS * STAGE_BYTES;       // [VB][128 state rows][128 B] rounded state, B operand of w S
  unsigned char *sOp = sS + VB * K * 128;              // [VB][64 tokens][128 B] B operand of k^T op
  unsigned char *sVn = sOp + VB * 8192;                // [VB][64 tokens][128 B] v_new, same layout (source of the tile store)
  float *sG = reinterpret_cast<float *>(sVn + VB * 8192);  // [2][64] gates
  __shared__ uint64_t full[NS], empty[NS], s_ready, p_done, op_ready, ds_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;
  __shared__ volatile int abort_snap[2];  // the flag as sampled by one thread before a barrier: the epilogue leaves as one

  const flab_args &a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&s_ready, EW);
    mbar_init(&p_done, 1);
    mbar_init(&op_ready, EW);
    mbar_init(&ds_done, 1);
    abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 256);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_base_s;

  const int vt = blockIdx.x, n = blockIdx.y / a.H, hd = blockIdx.y % a.H;
  const Seq s = seq_of(a, n);
  const int nt = s.nt, v0 = vt * BV;
  const bool use_g = a.g != nullptr;
  auto fail = [&](int code) {
    abort_flag = 1;
    atomicCAS(&tu_tc_error, 0, code);
  };

  if (warp == EW) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < nt && !abort_flag; ++i) {
        const int st = i % NS, ph = (i / NS) & 1;
        if (!mbar_wait(&empty[st], ph ^ 1)) { fail(41); break; }
        const int t0 = s.bos + i * C;
        unsigned char *wt = sStage + st * STAGE_BYTES, *kt = wt + KT_BYTES, *ut = kt + KT_BYTES;
        mbar_expect_tx(&full[st], STAGE_BYTES);
        const int c1 = a.head_first ? t0 : hd, c2 = a.head_first ? hd : t0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_4d(wt + j * 8192, &mapW, &full[st], 64 * j, c1, c2, s.b);
          tma_load_4d(kt + j * 8192, &mapK, &full[st], 64 * j, c1, c2, s.b);
        }
#pragma unroll
        for (int j = 0; j < VB; ++j) tma_load_4d(ut + j * 8192, &mapU, &full[st], v0 + 64 * j, c1, c2, s.b);
      }
    }
  } else if (warp == EW + 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_p = instr_desc(64, BV, p.ab_fmt, 0, 1);
      const uint32_t idesc_s = instr_desc(128, BV, p.ab_fmt, 1, 1);
      const uint64_t ds0 = desc_mnmajor(smem_u32(sS), 0, K * 128), do0 = desc_mnmajor(smem_u32(sOp), 0, 8192);
      for (int i = 0; i < nt && !abort_flag; ++i) {
        const int st = i % NS, ph = (i / NS) & 1, sp = i & 1;
        if (!mbar_wait(&full[st], ph)) { fail(42); break; }
        if (!mbar_wait(&s_ready, sp)) { fail(43); break; }
        fence_after_sync();
        const uint32_t wt = smem_u32(sStage + st * STAGE_BYTES), kt = wt + KT_BYTES;
        // descriptors differ from step to step only in the 16-byte-granular start address (low bits)
        const uint64_t dw0 = desc_kmajor(wt, 0, 8192), dk0 = desc_mnmajor(kt, 0, 8192);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma(tmem + TM_P, dw0 + (uint64_t)(((k >> 2) * 8192 + (k & 3) * 32) >> 4), ds0 + (uint64_t)((k * 2048) >> 4), idesc_p, k > 0);
        umma_commit(&p_done);
        if (!mbar_wait(&op_ready, sp)) { fail(44); break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem + TM_DS, dk0 + (uint64_t)((k * 2048) >> 4), do0 + (uint64_t)((k * 2048) >> 4), idesc_s, k > 0);
        umma_commit(&ds_done);
        umma_commit(&empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int wq = warp & 3, chh = warp >> 2, g8 = lane >> 2, t4 = lane & 3;  // lane quadrant, 32-column group
    const uint32_t lane_base = (uint32_t)(32 * wq) << 16;
    // phase A view: state row `srow`, columns [sc0, sc0 + NC)
    const int srow = 32 * wq + lane, sc0 = NC * chh;
    // phase B view: token rows row_lo / row_hi, columns 32 chh + 8 ni + 2 t4
    const int row_lo = 16 * wq + g8, row_hi = row_lo + 8;
    const size_t st_off = ((size_t)n * a.H + hd) * K * a.V + (size_t)srow * a.V + v0 + sc0;
    float S[NC];
    if (a.h0) {
      const float4 *src = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(a.h0) + st_off);
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) {
        const float4 x = src[j];
        S[4 * j] = x.x, S[4 * j + 1] = x.y, S[4 * j + 2] = x.z, S[4 * j + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j) S[j] = 0.f;
    }
    const float *G = use_g ? reinterpret_cast<const float *>(a.g) + tok_off(a, s, hd, 0, 1) : nullptr;
    const size_t gs = tok_stride(a, 1);
    auto gate_of = [&](int i) -> float { return (use_g && tid < C && i * C + tid < s.len) ? G[(size_t)(i * C + tid) * gs] : 0.f; };
    float g_pf = nt > 0 ? gate_of(0) : 0.f;
    float d_prev = 1.f;
    bf16 *vout = reinterpret_cast<bf16 *>(a.v_new);
    const size_t vs = tok_stride(a, a.V);
    bool ok = true;
    for (int i = 0; i <= nt; ++i) {
      const int sp = i & 1;
      // ---- phase A: S <- d S + dS of the previous chunk
      if (i > 0) {
        if (!mbar_wait(&ds_done, sp ^ 1)) { fail(45); ok = false; }
        fence_after_sync();
        float dS[32];
        tmem_ld_32x32b_x32(tmem + lane_base + TM_DS + sc0, dS);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) S[c] = fmaf(S[c], d_prev, dS[c]);
      }
      if (i == nt) break;
      {
        // rounded state -> swizzled tile: the B operand of the next product and the source of the h[t] tile store
#pragma unroll
        for (int cc = 0; cc < NC / 8; ++cc) {
          int4 x;
          if (p.ab_fmt) {
            __nv_bfloat162 *px = reinterpret_cast<__nv_bfloat162 *>(&x);
#pragma unroll
            for (int j = 0; j < 4; ++j) px[j] = __floats2bfloat162_rn(S[8 * cc + 2 * j], S[8 * cc + 2 * j + 1]);
          } else {
            __half2 *px = reinterpret_cast<__half2 *>(&x);
#pragma unroll
            for (int j = 0; j < 4; ++j) px[j] = __floats2half2_rn(S[8 * cc + 2 * j], S[8 * cc + 2 * j + 1]);
          }
          const int col = sc0 + 8 * cc;
          *reinterpret_cast<int4 *>(sS + (col >> 6) * (K * 128) + srow * 128 + ((((col & 63) >> 3) ^ (srow & 7)) << 4)) = x;
        }
      }
      if (tid < C) sG[sp * C + tid] = g_pf;
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_ready);
      if (tid == 0) {
        tma_store_wait_read();  // the v_new store of the previous chunk has read its tile
        abort_snap[0] = abort_flag;
      }
      named_barrier(1, ET);  // gates visible; the previous chunk's v_new store has drained its staging tile
      if (abort_snap[0]) break;
      if (tid == 0) {  // h[t]: one tile store per 64-column box, straight from the operand tile
#pragma unroll
        for (int j = 0; j < VB; ++j) tma_store_2d(&mapH, sS + j * (K * 128), v0 + 64 * j, ((s.c0 + i) * a.H + hd) * K);
        tma_store_commit();
      }
      if (i + 1 < nt) g_pf = gate_of(i + 1);
      const int rows = min(C, s.len - i * C), last = rows - 1;
      const float *gc = sG + sp * C;
      const float gl = gc[last];
      float e1_lo = 1.f, e1_hi = 1.f, e2_lo = 1.f, e2_hi = 1.f;
      if (use_g) {
        e1_lo = __expf(gc[row_lo]), e1_hi = __expf(gc[row_hi]);
        e2_lo = __expf(gl - gc[row_lo]), e2_hi = __expf(gl - gc[row_hi]);
        d_prev = __expf(gl);
      }
      if (row_lo >= rows) e2_lo = 0.f;  // rows past the end of the sequence contribute nothing to the state
      if (row_hi >= rows) e2_hi = 0.f;
      // ---- phase B: P = w S  ->  v_new, op
      const int st = i % NS, ph = (i / NS) & 1;
      if (!mbar_wait(&full[st], ph)) { fail(46); ok = false; }  // u tile (already complete: the product waited on it)
      if (!mbar_wait(&p_done, sp)) { fail(47); ok = false; }
      fence_after_sync();
      float pr[NC / 8][4];
      tmem_ld_frag<NC / 8>(tmem + lane_base + TM_P + NC * chh, pr);
      tmem_ld_wait();
      const unsigned char *ut = sStage + st * STAGE_BYTES + 2 * KT_BYTES;
#pragma unroll
      for (int ni = 0; ni < NC / 8; ++ni) {
        const int col = NC * chh + 8 * ni + 2 * t4;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int row = hf ? row_hi : row_lo;
          const uint32_t off = (uint32_t)(col >> 6) * 8192u + sw128_offset(row, col & 63);
          float u0, u1;
          if (p.ab_fmt) {
            const float2 uu = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(ut + off));
            u0 = uu.x, u1 = uu.y;
          } else {
            const float2 uu = __half22float2(*reinterpret_cast<const __half2 *>(ut + off));
            u0 = uu.x, u1 = uu.y;
          }
          const float e1 = hf ? e1_hi : e1_lo, e2 = hf ? e2_hi : e2_lo;
          const float x0 = u0 - e1 * pr[ni][2 * hf], x1 = u1 - e1 * pr[ni][2 * hf + 1];
          if (p.ab_fmt) {
            const __nv_bfloat162 vn = __floats2bfloat162_rn(x0, x1);
            *reinterpret_cast<__nv_bfloat162 *>(sVn + off) = vn;
            const float2 vr = __bfloat1622float2(vn);
            *reinterpret_cast<__nv_bfloat162 *>(sOp + off) = __floats2bfloat162_rn(vr.x * e2, vr.y * e2);
          } else {
            const __half2 vn = __floats2half2_rn(x0, x1);
            *reinterpret_cast<__half2 *>(sVn + off) = vn;
            const float2 vr = __half22float2(vn);
            *reinterpret_cast<__half2 *>(sOp + off) = __floats2half2_rn(vr.x * e2, vr.y * e2);
          }
        }
      }
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&op_ready);
      if (tid == 0) {
        tma_store_wait_read();  // the h[t] store has read the state tile: phase A of the next chunk may overwrite it
        abort_snap[1] = abort_flag;
      }
      named_barrier(1, ET);  // v_new tile complete
      if (abort_snap[1]) break;
      if (rows == C) {
        if (tid == 0) {
          const int t0 = s.bos + i * C, c1 = a.head_first ? t0 : hd, c2 = a.head_first ? hd : t0;
#pragma unroll
          for (int j = 0; j < VB; ++j) tma_store_4d(&mapVn, sVn + j * 8192, v0 + 64 * j, c1, c2, s.b);
          tma_store_commit();
        }
      } else {
        // ragged last chunk: a tile store would write past the end of the sequence
        bf16 *dst = vout + tok_off(a, s, hd, i * C, a.V) + v0;
        for (int e = tid; e < rows * (BV / 8); e += ET) {
          const int r_ = e / (BV / 8), c_ = (e - r_ * (BV / 8)) * 8;
          *reinterpret_cast<int4 *>(dst + (size_t)r_ * vs + c_) =
              *reinterpret_cast<const int4 *>(sVn + (c_ >> 6) * 8192 + sw128_offset(r_, c_ & 63));
        }
      }
    }
    if (tid == 0) tma_store_wait_all();
    if (ok && !abort_flag && a.ht) {
      float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.ht) + st_off);
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) dst[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

template <int VB, int NS> static int launch_tc_dh(const flab_args *a, cudaStream_t stream) {
  constexpr int BV = 64 * VB;
  CUtensorMap mW, mK, mU, mH, mVn;
  if (int e = make_token_map(&mW, a->w, a, a->K)) return e;
  if (int e = make_token_map(&mK, a->k, a, a->K)) return e;
  if (int e = make_token_map(&mU, a->u, a, a->V)) return e;
  if (int e = make_state_map(&mH, a->h, a, 128)) return e;
  if (int e = make_token_map(&mVn, a->v_new, a, a->V)) return e;
  TcDhParams p;
  p.a = *a;
  p.v_tiles = a->V / BV;
  p.ab_fmt = a->dtype == FLAB_BF16 ? 1 : 0;
  constexpr uint32_t STAGE = 2 * 16384 + VB * 8192;
  const size_t smem = 1024 + NS * (size_t)STAGE + (size_t)VB * 128 * 128 + 2 * (size_t)VB * 8192 + 2 * C * sizeof(float);
  auto kern = tc_delta_fwd_h_kernel<VB, NS>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<dim3(p.v_tiles, a->N * a->H), 64 * (4 * VB + 1), smem, stream>>>(mW, mK, mU, mH, mVn, p);
  return check_launch("delta_fwd_h(tc)");
}

// Returns 1 if the tcgen05 kernel took the call, 0 if the shape is outside its domain, < 0 on error.
int tc_delta_fwd_h_try(const flab_args *a, cudaStream_t stream) {
  if (a->dtype != FLAB_BF16 && a->dtype != FLAB_FP16) return 0;
  if (a->K != 128 || a->V % 64 != 0) return 0;
  const void *ptrs[5] = {a->k, a->w, a->u, a->h, a->v_new};
  for (int i = 0; i < 5; ++i)
    if (reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return 0;
  if ((a->h0 && reinterpret_cast<uintptr_t>(a->h0) % 16 != 0) || (a->ht && reinterpret_cast<uintptr_t>(a->ht) % 16 != 0)) return 0;
  const int rc = (a->V % 128 == 0) ? launch_tc_dh<2, 3>(a, stream) : launch_tc_dh<1, 4>(a, stream);
  return rc < 0 ? rc : 1;
}

}  // namespace flab
