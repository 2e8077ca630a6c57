// tcgen05 / TMA version of the delta-rule state scans (bf16 / fp16, K = 128, V % 64 == 0):
//   forward, per chunk t:  h[t] = S;  v_new = u - e^{b} (w S);  S <- e^{b_L} S + k^T (e^{b_L - b} v_new)
//   (fla/ops/common/chunk_delta_h.py:248-321)
//   backward, chunks in reverse:  dh[t] = S;  dv2 = dv + e^{b_L - b} (k S);
//                                 S <- e^{b_L} S + q^T (scale e^{b} do) - w^T (e^{b} dv2)
//   (fla/ops/common/chunk_delta_h.py:323-423)
// and of the plain chunk-state scans S <- e^{b_L} S + k^T (e^{b_L-b} v), dS <- e^{b_L} dS + q^T (scale e^{b} do)
// (fla/ops/common/chunk_h.py:42-122, 125-215; scalar gate or none), which are the same chain without the
// dependent product.
// The directions share one kernel: "P" below is the dependent product against the rounded state
// (forward w S, backward k S), "y" the tile it corrects (u -> v_new, dv -> dv2), "op" the gate-scaled
// operand of the state update.
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
  int state_only;  // delta modes: h / v_new (dh / dv2) are not stored, only the final state
};

enum { DH_FWD = 0, DH_BWD = 1, DH_SIMPLE_FWD = 2, DH_SIMPLE_BWD = 3, DH_GK_FWD = 4, DH_GK_BWD = 5 };

template <int VB /* BV / 64 */, int NS, int MODE>
__global__ void __launch_bounds__(64 * (4 * VB + 1), 1)
tc_delta_h_kernel(const __grid_constant__ CUtensorMap mapA1, const __grid_constant__ CUtensorMap mapA2,
                  const __grid_constant__ CUtensorMap mapA3, const __grid_constant__ CUtensorMap mapY,
                  const __grid_constant__ CUtensorMap mapDo, const __grid_constant__ CUtensorMap mapH,
                  const __grid_constant__ CUtensorMap mapYo, const TcDhParams p) {
  // tensor maps: A1 = A operand of P (fwd w, bwd k; simple: the transposed A operand of the update, k or q);
  // A2, A3 = transposed A operands of the update (fwd k, -; bwd q, w); Y = corrected tile (fwd u, bwd dv; simple:
  // v or do); Do = do (bwd); H = h / dh (store); Yo = v_new / dv2 (store)
  using namespace tc;
  constexpr int K = 128, BV = 64 * VB, NC = 32;  // NC: state columns per epilogue thread
  constexpr int EW = BV / 8, ET = 32 * EW;         // epilogue warps (4 lane quadrants x BV/32 column groups), threads
  constexpr bool BWD = (MODE & 1) != 0, SIMPLE = MODE >= 2, GK = MODE >= 4;  // GK: simple scan with a gate per key channel
  constexpr int NKT = SIMPLE ? 1 : (BWD ? 3 : 2), NVT = (BWD && !SIMPLE) ? 2 : 1;  // [tokens x K] and [tokens x BV] tiles per chunk
  constexpr uint32_t KT_BYTES = 2 * 8192, U_BYTES = VB * 8192, STAGE_BYTES = NKT * KT_BYTES + NVT * U_BYTES;
  constexpr uint32_t TM_DS = 0, TM_P = 128;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sStage = base;                        // [NS][A1 | A2 (| A3) | y (| do)]
  unsigned char *sS = sStage + NS * STAGE_BYTES;       // [VB][128 state rows][128 B] rounded state, B operand of w S
  unsigned char *sOp = sS + VB * K * 128;              // [VB][64 tokens][128 B] B operand of k^T op
  unsigned char *sVn = sOp + VB * 8192;                // [VB][64 tokens][128 B] v_new, same layout (source of the tile store)
  float *sG = reinterpret_cast<float *>(sVn + VB * 8192);  // [2][64] gates ([2][128]: the last row's gates per channel, GK)
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
        const int t0 = s.bos + (BWD ? nt - 1 - i : i) * C;
        unsigned char *t1 = sStage + st * STAGE_BYTES, *yt = t1 + NKT * KT_BYTES;
        mbar_expect_tx(&full[st], STAGE_BYTES);
        const int c1 = a.head_first ? t0 : hd, c2 = a.head_first ? hd : t0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tma_load_4d(t1 + j * 8192, &mapA1, &full[st], 64 * j, c1, c2, s.b);
          if (NKT > 1) tma_load_4d(t1 + KT_BYTES + j * 8192, &mapA2, &full[st], 64 * j, c1, c2, s.b);
          if (NKT > 2) tma_load_4d(t1 + 2 * KT_BYTES + j * 8192, &mapA3, &full[st], 64 * j, c1, c2, s.b);
        }
#pragma unroll
        for (int j = 0; j < VB; ++j) {
          tma_load_4d(yt + j * 8192, &mapY, &full[st], v0 + 64 * j, c1, c2, s.b);
          if (NVT > 1) tma_load_4d(yt + U_BYTES + j * 8192, &mapDo, &full[st], v0 + 64 * j, c1, c2, s.b);
        }
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
        const uint32_t t1 = smem_u32(sStage + st * STAGE_BYTES), t2 = SIMPLE ? t1 : t1 + KT_BYTES, t3 = t2 + KT_BYTES;
        // descriptors differ from step to step only in the 16-byte-granular start address (low bits)
        const uint64_t d1 = desc_kmajor(t1, 0, 8192), d2 = desc_mnmajor(t2, 0, 8192);
        if (!SIMPLE) {
          if (!mbar_wait(&s_ready, sp)) { fail(43); break; }
          fence_after_sync();
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma(tmem + TM_P, d1 + (uint64_t)(((k >> 2) * 8192 + (k & 3) * 32) >> 4), ds0 + (uint64_t)((k * 2048) >> 4), idesc_p, k > 0);
          umma_commit(&p_done);
        }
        if (!mbar_wait(&op_ready, sp)) { fail(44); break; }
        fence_after_sync();
        if (GK) {
          // (k e^{b_L-b})^T v or (scale q e^{b})^T do: the key tile was rescaled in place, the value tile is used as loaded
          const uint64_t dy = desc_mnmajor(t1 + NKT * KT_BYTES, 0, 8192);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem + TM_DS, d2 + (uint64_t)((k * 2048) >> 4), dy + (uint64_t)((k * 2048) >> 4), idesc_s, k > 0);
        } else if (!BWD || SIMPLE) {
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem + TM_DS, d2 + (uint64_t)((k * 2048) >> 4), do0 + (uint64_t)((k * 2048) >> 4), idesc_s, k > 0);
        } else {
          // q^T (scale e^{b} do): the do tile was rescaled in place by the epilogue; then w^T (-e^{b} dv2)
          const uint64_t d3 = desc_mnmajor(t3, 0, 8192), dd = desc_mnmajor(t1 + NKT * KT_BYTES + U_BYTES, 0, 8192);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem + TM_DS, d2 + (uint64_t)((k * 2048) >> 4), dd + (uint64_t)((k * 2048) >> 4), idesc_s, k > 0);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem + TM_DS, d3 + (uint64_t)((k * 2048) >> 4), do0 + (uint64_t)((k * 2048) >> 4), idesc_s, 1);
        }
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
    const float *S0 = reinterpret_cast<const float *>(BWD ? a.dht : a.h0);  // same slots in every mode
    float *S1 = reinterpret_cast<float *>(BWD ? a.dh0 : a.ht);
    if (S0) {
      const float4 *src = reinterpret_cast<const float4 *>(S0 + st_off);
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
    // i counts processed chunks; the backward scan walks them in reverse
    auto chunk_at = [&](int i) { return BWD ? nt - 1 - i : i; };
    auto gate_of = [&](int i) -> float {
      const int t = chunk_at(i) * C + tid;
      return (use_g && tid < C && t < s.len) ? G[(size_t)t * gs] : 0.f;
    };
    // GK: gates [tokens][K] fp32; the last row of the chunk (decay of the state rows) goes through shared memory,
    // the factors of this thread's 16 key-tile elements are fetched a chunk ahead into registers
    const float *GKp = GK ? reinterpret_cast<const float *>(a.gk) + tok_off(a, s, hd, 0, K) : nullptr;
    const size_t gks = tok_stride(a, K);
    auto gk_last_of = [&](int i) -> float {
      const int it_ = chunk_at(i), t = it_ * C + min(C, s.len - it_ * C) - 1;
      return tid < K ? GKp[(size_t)t * gks + tid] : 0.f;
    };
    float2 gk_pf[2][NC / 8];
    auto gk_load = [&](int i) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int t = chunk_at(i) * C + (hf ? row_hi : row_lo);
#pragma unroll
        for (int ni = 0; ni < NC / 8; ++ni)
          gk_pf[hf][ni] = t < s.len ? *reinterpret_cast<const float2 *>(GKp + (size_t)t * gks + NC * chh + 8 * ni + 2 * t4) : make_float2(0.f, 0.f);
      }
    };
    float g_pf = nt > 0 ? (GK ? gk_last_of(0) : gate_of(0)) : 0.f;
    if (GK && nt > 0) gk_load(0);
    float d_prev = 1.f;
    bf16 *vout = reinterpret_cast<bf16 *>(BWD ? a.dv2 : a.v_new);
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
      if (GK) {
        if (tid < K) sG[sp * K + tid] = g_pf;
      } else if (tid < C) sG[sp * C + tid] = g_pf;
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (!SIMPLE && lane == 0) mbar_arrive(&s_ready);
      if (tid == 0) {
        tma_store_wait_read();  // the v_new store of the previous chunk has read its tile
        abort_snap[0] = abort_flag;
      }
      named_barrier(1, ET);  // gates visible; the previous chunk's v_new store has drained its staging tile
      if (abort_snap[0]) break;
      if (tid == 0 && !p.state_only) {  // h[t]: one tile store per 64-column box, straight from the operand tile
#pragma unroll
        for (int j = 0; j < VB; ++j) tma_store_2d(&mapH, sS + j * (K * 128), v0 + 64 * j, ((s.c0 + chunk_at(i)) * a.H + hd) * K);
        tma_store_commit();
      }
      if (i + 1 < nt) g_pf = GK ? gk_last_of(i + 1) : gate_of(i + 1);
      const int it = chunk_at(i), rows = min(C, s.len - it * C), last = rows - 1;
      const float *gc = sG + sp * (GK ? K : C);
      const float gl = GK ? 0.f : gc[last];
      // row factors: fa multiplies P, fo turns the corrected tile into op
      //   forward : v_new = u - e^{b} P,         op = e^{b_L-b} v_new
      //   backward: dv2   = dv + e^{b_L-b} P,    op = -e^{b} dv2,   do' = scale e^{b} do
      float e1_lo = 1.f, e1_hi = 1.f, e2_lo = 1.f, e2_hi = 1.f;
      if (GK) d_prev = __expf(gc[srow]);
      if (use_g && !GK) {
        e1_lo = __expf(gc[row_lo]), e1_hi = __expf(gc[row_hi]);
        e2_lo = __expf(gl - gc[row_lo]), e2_hi = __expf(gl - gc[row_hi]);
        d_prev = __expf(gl);
      }
      const bool in_lo = row_lo < rows, in_hi = row_hi < rows;  // rows past the end of the sequence add nothing to the state
      //   simple  : op = e^{b_L-b} v (forward), op = scale e^{b} do (backward)
      const float fa_lo = BWD ? e2_lo : -e1_lo, fa_hi = BWD ? e2_hi : -e1_hi;
      float fo_lo = BWD ? -e1_lo : e2_lo, fo_hi = BWD ? -e1_hi : e2_hi;
      if (SIMPLE && BWD) fo_lo = e1_lo * a.scale, fo_hi = e1_hi * a.scale;
      if (!in_lo) fo_lo = 0.f;
      if (!in_hi) fo_hi = 0.f;
      // ---- phase B: P -> corrected tile y', op
      const int st = i % NS, ph = (i / NS) & 1;
      if (!mbar_wait(&full[st], ph)) { fail(46); ok = false; }  // y (and do) tiles (already complete: the product waited on it)
      unsigned char *yt = sStage + st * STAGE_BYTES + NKT * KT_BYTES;
      if (BWD && !SIMPLE) {
        // do' = scale e^{b} do, in place (runs while the tensor core computes P)
        unsigned char *dt = yt + U_BYTES;
        const float s_lo = in_lo ? e1_lo * a.scale : 0.f, s_hi = in_hi ? e1_hi * a.scale : 0.f;
#pragma unroll
        for (int ni = 0; ni < NC / 8; ++ni) {
          const int col = NC * chh + 8 * ni + 2 * t4;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const uint32_t off = (uint32_t)(col >> 6) * 8192u + sw128_offset(hf ? row_hi : row_lo, col & 63);
            const float f = hf ? s_hi : s_lo;
            if (p.ab_fmt) {
              __nv_bfloat162 *q2 = reinterpret_cast<__nv_bfloat162 *>(dt + off);
              const float2 x = __bfloat1622float2(*q2);
              *q2 = __floats2bfloat162_rn(x.x * f, x.y * f);
            } else {
              __half2 *q2 = reinterpret_cast<__half2 *>(dt + off);
              const float2 x = __half22float2(*q2);
              *q2 = __floats2half2_rn(x.x * f, x.y * f);
            }
          }
        }
      }
      if (GK) {
        // key tile rescaled in place: k e^{b_L-b} (forward), scale q e^{b} (backward); rows past the end are zeroed
        unsigned char *kt = sStage + st * STAGE_BYTES;
#pragma unroll
        for (int ni = 0; ni < NC / 8; ++ni) {
          const int col = NC * chh + 8 * ni + 2 * t4;
          const float gl0 = gc[col], gl1 = gc[col + 1];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const uint32_t off = (uint32_t)(col >> 6) * 8192u + sw128_offset(hf ? row_hi : row_lo, col & 63);
            const float2 bb = gk_pf[hf][ni];
            float f0, f1;
            if (BWD) f0 = a.scale * __expf(bb.x), f1 = a.scale * __expf(bb.y);
            else f0 = __expf(gl0 - bb.x), f1 = __expf(gl1 - bb.y);
            if (!(hf ? in_hi : in_lo)) f0 = f1 = 0.f;
            if (p.ab_fmt) {
              __nv_bfloat162 *q2 = reinterpret_cast<__nv_bfloat162 *>(kt + off);
              const float2 x = __bfloat1622float2(*q2);
              *q2 = __floats2bfloat162_rn(x.x * f0, x.y * f1);
            } else {
              __half2 *q2 = reinterpret_cast<__half2 *>(kt + off);
              const float2 x = __half22float2(*q2);
              *q2 = __floats2half2_rn(x.x * f0, x.y * f1);
            }
          }
        }
        if (i + 1 < nt) gk_load(i + 1);
      }
      float pr[NC / 8][4];
      if (!SIMPLE) {
        if (!mbar_wait(&p_done, sp)) { fail(47); ok = false; }
        fence_after_sync();
        tmem_ld_frag<NC / 8>(tmem + lane_base + TM_P + NC * chh, pr);
        tmem_ld_wait();
      }
#pragma unroll
      for (int ni = 0; ni < (GK ? 0 : NC / 8); ++ni) {
        const int col = NC * chh + 8 * ni + 2 * t4;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int row = hf ? row_hi : row_lo;
          const uint32_t off = (uint32_t)(col >> 6) * 8192u + sw128_offset(row, col & 63);
          float u0, u1;
          if (p.ab_fmt) {
            const float2 uu = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(yt + off));
            u0 = uu.x, u1 = uu.y;
          } else {
            const float2 uu = __half22float2(*reinterpret_cast<const __half2 *>(yt + off));
            u0 = uu.x, u1 = uu.y;
          }
          const float fa = hf ? fa_hi : fa_lo, fo = hf ? fo_hi : fo_lo;
          if (SIMPLE) {
            if (p.ab_fmt) *reinterpret_cast<__nv_bfloat162 *>(sOp + off) = __floats2bfloat162_rn(u0 * fo, u1 * fo);
            else *reinterpret_cast<__half2 *>(sOp + off) = __floats2half2_rn(u0 * fo, u1 * fo);
            continue;
          }
          const float x0 = fmaf(fa, pr[ni][2 * hf], u0), x1 = fmaf(fa, pr[ni][2 * hf + 1], u1);
          if (p.ab_fmt) {
            const __nv_bfloat162 vn = __floats2bfloat162_rn(x0, x1);
            *reinterpret_cast<__nv_bfloat162 *>(sVn + off) = vn;
            const float2 vr = __bfloat1622float2(vn);
            *reinterpret_cast<__nv_bfloat162 *>(sOp + off) = __floats2bfloat162_rn(vr.x * fo, vr.y * fo);
          } else {
            const __half2 vn = __floats2half2_rn(x0, x1);
            *reinterpret_cast<__half2 *>(sVn + off) = vn;
            const float2 vr = __half22float2(vn);
            *reinterpret_cast<__half2 *>(sOp + off) = __floats2half2_rn(vr.x * fo, vr.y * fo);
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
      if (SIMPLE || p.state_only) continue;  // no corrected tile to store
      if (rows == C) {
        if (tid == 0) {
          const int t0 = s.bos + it * C, c1 = a.head_first ? t0 : hd, c2 = a.head_first ? hd : t0;
#pragma unroll
          for (int j = 0; j < VB; ++j) tma_store_4d(&mapYo, sVn + j * 8192, v0 + 64 * j, c1, c2, s.b);
          tma_store_commit();
        }
      } else {
        // ragged last chunk: a tile store would write past the end of the sequence
        bf16 *dst = vout + tok_off(a, s, hd, it * C, a.V) + v0;
        for (int e = tid; e < rows * (BV / 8); e += ET) {
          const int r_ = e / (BV / 8), c_ = (e - r_ * (BV / 8)) * 8;
          *reinterpret_cast<int4 *>(dst + (size_t)r_ * vs + c_) =
              *reinterpret_cast<const int4 *>(sVn + (c_ >> 6) * 8192 + sw128_offset(r_, c_ & 63));
        }
      }
    }
    if (tid == 0) tma_store_wait_all();
    if (ok && !abort_flag && S1) {
      float4 *dst = reinterpret_cast<float4 *>(S1 + st_off);
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) dst[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

template <int VB, int NS, int MODE> static int launch_tc_dh(const flab_args *a, cudaStream_t stream) {
  constexpr int BV = 64 * VB;
  constexpr bool BWD = (MODE & 1) != 0, SIMPLE = MODE >= 2, GK = MODE >= 4;
  CUtensorMap mA1, mA2, mA3, mY, mDo, mH, mYo;
  const void *a1 = SIMPLE ? (BWD ? a->q : a->k) : (BWD ? a->k : a->w);
  const void *y = SIMPLE ? (BWD ? a->d_o : a->v) : (BWD ? a->dv : a->u);
  if (int e = make_token_map(&mA1, a1, a, a->K)) return e;
  if (int e = make_token_map(&mA2, SIMPLE ? a1 : (BWD ? a->q : a->k), a, a->K)) return e;
  if (int e = make_token_map(&mA3, (BWD && !SIMPLE) ? a->w : a1, a, a->K)) return e;
  // state-only forward scan: u may be narrower than the state (S = its columns); the tile loads past its last
  // column are filled with zeros by the copy engine
  const int ycols = (!SIMPLE && !BWD && (a->flags & FLAB_F_STATE_ONLY) && a->S > 0) ? a->S : a->V;
  if (int e = make_token_map(&mY, y, a, ycols)) return e;
  if (int e = make_token_map(&mDo, (BWD && !SIMPLE) ? a->d_o : y, a, a->V)) return e;
  // a state-only scan stores neither: the maps are still encoded (over a tensor of the right element type) and never used
  const bool state_only = !SIMPLE && (a->flags & FLAB_F_STATE_ONLY) != 0;
  if (int e = make_state_map(&mH, state_only ? a->k : (BWD ? a->dh : a->h), a, 128)) return e;
  if (int e = make_token_map(&mYo, (SIMPLE || state_only) ? y : (BWD ? a->dv2 : a->v_new), a, a->V)) return e;
  TcDhParams p;
  p.a = *a;
  p.v_tiles = a->V / BV;
  p.ab_fmt = a->dtype == FLAB_BF16 ? 1 : 0;
  p.state_only = state_only ? 1 : 0;
  constexpr int NKT = SIMPLE ? 1 : (BWD ? 3 : 2), NVT = (BWD && !SIMPLE) ? 2 : 1;
  constexpr uint32_t STAGE = NKT * 16384 + NVT * VB * 8192;
  const size_t smem = 1024 + NS * (size_t)STAGE + (size_t)VB * 128 * 128 + 2 * (size_t)VB * 8192 + 2 * (GK ? 128 : C) * sizeof(float);
  auto kern = tc_delta_h_kernel<VB, NS, MODE>;
  if (int e = set_smem(kern, smem)) return e;
  kern<<<dim3(p.v_tiles, a->N * a->H), 64 * (4 * VB + 1), smem, stream>>>(mA1, mA2, mA3, mY, mDo, mH, mYo, p);
  return check_launch(SIMPLE ? (BWD ? "chunk_bwd_dh(tc)" : "chunk_fwd_h(tc)") : (BWD ? "delta_bwd_dhu(tc)" : "delta_fwd_h(tc)"));
}

static bool tc_dh_ok(const flab_args *a, const void *const *ptrs, int n) {
  if (a->dtype != FLAB_BF16 && a->dtype != FLAB_FP16) return false;
  if (a->K != 128 || a->V % 64 != 0) return false;
  if ((unsigned long long)a->NT * a->H * a->K >= (1ull << 31)) return false;  // tile coordinates of the state tensor are 32-bit
  for (int i = 0; i < n; ++i)
    if (ptrs[i] && reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return false;
  return true;
}

// Return 1 if the tcgen05 kernel took the call, 0 if the shape is outside its domain, < 0 on error.
int tc_delta_fwd_h_try(const flab_args *a, cudaStream_t stream) {
  const void *ptrs[7] = {a->k, a->w, a->u, a->h, a->v_new, a->h0, a->ht};
  if (!tc_dh_ok(a, ptrs, 7)) return 0;
  const int rc = (a->V % 128 == 0) ? launch_tc_dh<2, 3, DH_FWD>(a, stream) : launch_tc_dh<1, 4, DH_FWD>(a, stream);
  return rc < 0 ? rc : 1;
}

int tc_delta_bwd_dhu_try(const flab_args *a, cudaStream_t stream) {
  const void *ptrs[9] = {a->q, a->k, a->w, a->d_o, a->dv, a->dh, a->dv2, a->dht, a->dh0};
  if (!tc_dh_ok(a, ptrs, 9)) return 0;
  const int rc = (a->V % 128 == 0) ? launch_tc_dh<2, 2, DH_BWD>(a, stream) : launch_tc_dh<1, 3, DH_BWD>(a, stream);
  return rc < 0 ? rc : 1;
}

// Plain chunk-state scans: no gate, a scalar gate per (token, head), or a gate per key channel (GLA).
int tc_chunk_fwd_h_try(const flab_args *a, cudaStream_t stream) {
  if (a->gv || (a->gk && a->g)) return 0;
  const void *ptrs[6] = {a->k, a->v, a->h, a->h0, a->ht, a->gk};
  if (!tc_dh_ok(a, ptrs, 6)) return 0;
  if (a->gk) {
    if (a->V % 128 != 0) return 0;  // the 16 epilogue warps of the 128-column tile cover the [64][128] key tile
    const int rc = launch_tc_dh<2, 4, DH_GK_FWD>(a, stream);
    return rc < 0 ? rc : 1;
  }
  const int rc = (a->V % 128 == 0) ? launch_tc_dh<2, 4, DH_SIMPLE_FWD>(a, stream) : launch_tc_dh<1, 4, DH_SIMPLE_FWD>(a, stream);
  return rc < 0 ? rc : 1;
}

int tc_chunk_bwd_dh_try(const flab_args *a, cudaStream_t stream) {
  if (a->gv || (a->gk && a->g)) return 0;
  const void *ptrs[6] = {a->q, a->d_o, a->dh, a->dht, a->dh0, a->gk};
  if (!tc_dh_ok(a, ptrs, 6)) return 0;
  if (a->gk) {
    if (a->V % 128 != 0) return 0;
    const int rc = launch_tc_dh<2, 4, DH_GK_BWD>(a, stream);
    return rc < 0 ? rc : 1;
  }
  const int rc = (a->V % 128 == 0) ? launch_tc_dh<2, 4, DH_SIMPLE_BWD>(a, stream) : launch_tc_dh<1, 4, DH_SIMPLE_BWD>(a, stream);
  return rc < 0 ? rc : 1;
}

}  // namespace flab
