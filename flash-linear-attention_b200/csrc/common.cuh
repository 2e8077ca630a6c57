// Shared device helpers: element types, sequence/chunk addressing, shared-memory tile movement
// and the warp-level tile GEMM (mma.sync for 16-bit types, FFMA for fp32).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flab200.h"

namespace flab {

constexpr int C = FLAB_CHUNK;  // tokens per chunk

typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------------------------------------
// element type traits
// ------------------------------------------------------------------------------------------------
template <typename T> struct Num;
template <> struct Num<bf16> {
  static constexpr int id = FLAB_BF16;
  static constexpr int pad = 8;  // extra elements per shared-memory row (keeps ldmatrix conflict free)
  __device__ __forceinline__ static float f(bf16 x) { return __bfloat162float(x); }
  __device__ __forceinline__ static bf16 t(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Num<__half> {
  static constexpr int id = FLAB_FP16;
  static constexpr int pad = 8;
  __device__ __forceinline__ static float f(__half x) { return __half2float(x); }
  __device__ __forceinline__ static __half t(float x) { return __float2half_rn(x); }
};
template <> struct Num<float> {
  static constexpr int id = FLAB_FP32;
  static constexpr int pad = 4;
  __device__ __forceinline__ static float f(float x) { return x; }
  __device__ __forceinline__ static float t(float x) { return x; }
};

// round a float through the element type (the reference rounds MMA operands to the input dtype)
template <typename T> __device__ __forceinline__ float rnd(float x) { return Num<T>::f(Num<T>::t(x)); }

__host__ __device__ __forceinline__ int round_up(int x, int m) { return (x + m - 1) / m * m; }
__host__ __device__ __forceinline__ int cdiv(int x, int m) { return (x + m - 1) / m; }

// exp(x) for x <= 0, else 0 (fla/ops/utils/exp.py:8)
__device__ __forceinline__ float safe_exp(float x) { return x <= 0.f ? expf(x) : 0.f; }

// ------------------------------------------------------------------------------------------------
// sequence / chunk addressing
// ------------------------------------------------------------------------------------------------
struct Seq {
  int b;    // batch row holding the sequence
  int bos;  // first token inside that row
  int len;  // tokens
  int nt;   // chunks
  int c0;   // global index of its first chunk
};

__device__ __forceinline__ Seq seq_of(const flab_args &a, int n) {
  Seq s;
  if (a.cu_seqlens) {
    s.b = 0;
    s.bos = a.cu_seqlens[n];
    s.len = a.cu_seqlens[n + 1] - s.bos;
    s.c0 = a.chunk_offsets[n];
  } else {
    s.b = n;
    s.bos = 0;
    s.len = a.T;
    s.c0 = n * cdiv(a.T, C);
  }
  s.nt = cdiv(s.len, C);
  return s;
}

// (sequence, chunk in sequence) of global chunk `c`
__device__ __forceinline__ void chunk_of(const flab_args &a, int c, int &n, int &it) {
  if (a.cu_seqlens) {
    n = a.chunk_indices[2 * c];
    it = a.chunk_indices[2 * c + 1];
  } else {
    int nts = cdiv(a.T, C);
    n = c / nts;
    it = c - n * nts;
  }
}

// element offset of (token t of sequence s, head h) in a token-major tensor with inner extent D
__device__ __forceinline__ size_t tok_off(const flab_args &a, const Seq &s, int h, int t, int D) {
  if (a.head_first) return (((size_t)s.b * a.H + h) * a.T + (size_t)(s.bos + t)) * D;
  return (((size_t)s.b * a.T + (size_t)(s.bos + t)) * a.H + h) * D;
}
__device__ __forceinline__ size_t tok_stride(const flab_args &a, int D) {
  return a.head_first ? (size_t)D : (size_t)a.H * D;
}

// ------------------------------------------------------------------------------------------------
// cp.async
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ------------------------------------------------------------------------------------------------
// tile movement: global <-> shared
// ------------------------------------------------------------------------------------------------
// Load `rows_total` rows x DP columns into s[r*ld + c]; element (r,c) comes from g[r*rstride + c]
// when r < rows_valid and c < D and is zero otherwise.  Uses 16-byte cp.async when addresses allow,
// scalar loads otherwise; the caller must cp_async_commit / wait and __syncthreads before use.
template <typename T>
__device__ __forceinline__ void tile_load(T *s, int ld, const T *g, size_t rstride, int rows_valid, int rows_total, int D,
                                          int DP, int tid, int nthreads) {
  constexpr int EPV = 16 / sizeof(T);
  const bool vec = (D % EPV == 0) && ((rstride * sizeof(T)) % 16 == 0) && (((uintptr_t)g) % 16 == 0);
  if (vec) {
    const int cpr = DP / EPV;  // 16-byte pieces per row
    if ((cpr & (cpr - 1)) == 0) {
      // power-of-two row length (the common case): shifts instead of divisions
      const int sh = 31 - __clz(cpr);
      for (int i = tid; i < (rows_total << sh); i += nthreads) {
        const int r = i >> sh, c = (i & (cpr - 1)) * EPV;
        const bool ok = (r < rows_valid) && (c < D);
        cp_async16(s + r * ld + c, ok ? (g + (size_t)r * rstride + c) : g, ok);
      }
    } else {
      for (int i = tid; i < rows_total * cpr; i += nthreads) {
        int r = i / cpr, c = (i - r * cpr) * EPV;
        bool ok = (r < rows_valid) && (c < D);
        const T *src = ok ? (g + (size_t)r * rstride + c) : g;
        cp_async16(s + r * ld + c, src, ok);
      }
    }
  } else {
    for (int i = tid; i < rows_total * DP; i += nthreads) {
      int r = i / DP, c = i - r * DP;
      T val = Num<T>::t(0.f);
      if (r < rows_valid && c < D) val = g[(size_t)r * rstride + c];
      s[r * ld + c] = val;
    }
  }
}

// Store rows_valid rows x D columns from s to g (16-byte vectors when possible).
template <typename T>
__device__ __forceinline__ void tile_store(T *g, size_t rstride, const T *s, int ld, int rows_valid, int D, int tid,
                                           int nthreads) {
  constexpr int EPV = 16 / sizeof(T);
  const bool vec = (D % EPV == 0) && ((rstride * sizeof(T)) % 16 == 0) && (((uintptr_t)g) % 16 == 0);
  if (vec) {
    const int cpr = D / EPV;
    if ((cpr & (cpr - 1)) == 0) {
      const int sh = 31 - __clz(cpr);
      for (int i = tid; i < (rows_valid << sh); i += nthreads) {
        const int r = i >> sh, c = (i & (cpr - 1)) * EPV;
        *reinterpret_cast<int4 *>(g + (size_t)r * rstride + c) = *reinterpret_cast<const int4 *>(s + r * ld + c);
      }
    } else {
      for (int i = tid; i < rows_valid * cpr; i += nthreads) {
        int r = i / cpr, c = (i - r * cpr) * EPV;
        *reinterpret_cast<int4 *>(g + (size_t)r * rstride + c) = *reinterpret_cast<const int4 *>(s + r * ld + c);
      }
    }
  } else {
    for (int i = tid; i < rows_valid * D; i += nthreads) {
      int r = i / D, c = i - r * D;
      g[(size_t)r * rstride + c] = s[r * ld + c];
    }
  }
}

// exp for gate factors: accurate expf for fp32 inputs (1e-5 parity bar), hardware exp2 path otherwise
template <typename T> __device__ __forceinline__ float fexp(float x) { return sizeof(T) == 4 ? expf(x) : __expf(x); }
template <typename T> __device__ __forceinline__ float safe_fexp(float x) { return x <= 0.f ? fexp<T>(x) : 0.f; }

// sum over a [rows x cols] window of a[r][c] * b[r][c] for two shared-memory tiles with the same leading
// dimension; cols and ld must be multiples of 16 bytes worth of elements (true for padded tiles)
template <typename T>
__device__ __forceinline__ float tile_dot(const T *a, const T *b, int ld, int rows, int cols, int tid, int nthreads) {
  constexpr int EPV = 16 / sizeof(T);
  const int cpr = cols / EPV;
  float acc = 0.f;
  for (int i = tid; i < rows * cpr; i += nthreads) {
    const int r = i / cpr, c = (i - r * cpr) * EPV;
    const int4 xa = *reinterpret_cast<const int4 *>(a + r * ld + c), xb = *reinterpret_cast<const int4 *>(b + r * ld + c);
    const T *pa = reinterpret_cast<const T *>(&xa), *pb = reinterpret_cast<const T *>(&xb);
#pragma unroll
    for (int j = 0; j < EPV; ++j) acc = fmaf(Num<T>::f(pa[j]), Num<T>::f(pb[j]), acc);
  }
  return acc;
}

// 64 per-token scalars (fp32) of one chunk -> shared; rows past the sequence end read as `fill`.
__device__ __forceinline__ void vec_load_f32(float *s, const float *g, size_t stride, int rows_valid, float fill,
                                             int tid, int nthreads) {
  for (int i = tid; i < C; i += nthreads) s[i] = (i < rows_valid) ? g[(size_t)i * stride] : fill;
}

// ------------------------------------------------------------------------------------------------
// warp tile GEMM.  acc[mi][ni][r] is the mma.sync m16n8 accumulator fragment:
//   row = m0 + 16*mi + (lane>>2) + 8*(r>>1),  col = n0 + 8*ni + 2*(lane&3) + (r&1)
// A_T = false: A(m,k) at A[m*lda + k];  A_T = true: A(m,k) at A[k*lda + m]
// B_KN = true: B(k,n) at B[k*ldb + n];  B_KN = false: B(k,n) at B[n*ldb + k]
// kdim must be a multiple of 16 for the 16-bit types (pad with zeros).
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void *p) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void *p) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<bf16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MI, int NI, bool A_T, bool B_KN, typename T> struct WarpGemm {
  static_assert(NI % 2 == 0, "NI must be even");
  __device__ __forceinline__ static void run(float (&acc)[MI][NI][4], const T *A, int lda, int m0, const T *B,
                                             int ldb, int n0, int kdim) {
    const int lane = threadIdx.x & 31;
    const int r = lane & 7, j = lane >> 3;
    for (int k0 = 0; k0 < kdim; k0 += 16) {
      uint32_t af[MI][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi) {
        if (!A_T) {
          ldsm4(af[mi], A + (size_t)(m0 + mi * 16 + (lane & 15)) * lda + k0 + ((lane >> 4) << 3));
        } else {
          ldsm4t(af[mi], A + (size_t)(k0 + r + ((j >> 1) << 3)) * lda + m0 + mi * 16 + ((j & 1) << 3));
        }
      }
#pragma unroll
      for (int np = 0; np < NI / 2; ++np) {
        uint32_t bfr[4];
        if (!B_KN) {
          ldsm4(bfr, B + (size_t)(n0 + np * 16 + ((j >> 1) << 3) + r) * ldb + k0 + ((j & 1) << 3));
        } else {
          ldsm4t(bfr, B + (size_t)(k0 + ((j & 1) << 3) + r) * ldb + n0 + np * 16 + ((j >> 1) << 3));
        }
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
          mma16816<T>(acc[mi][2 * np], af[mi], bfr[0], bfr[1]);
          mma16816<T>(acc[mi][2 * np + 1], af[mi], bfr[2], bfr[3]);
        }
      }
    }
  }
};

// fp32 operands: plain FFMA with the same accumulator layout (true IEEE fp32, no TF32).
template <int MI, int NI, bool A_T, bool B_KN> struct WarpGemm<MI, NI, A_T, B_KN, float> {
  __device__ __forceinline__ static void run(float (&acc)[MI][NI][4], const float *A, int lda, int m0,
                                             const float *B, int ldb, int n0, int kdim) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    for (int k = 0; k < kdim; ++k) {
      float a_lo[MI], a_hi[MI];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi) {
        int m = m0 + mi * 16 + g;
        a_lo[mi] = A_T ? A[(size_t)k * lda + m] : A[(size_t)m * lda + k];
        a_hi[mi] = A_T ? A[(size_t)k * lda + m + 8] : A[(size_t)(m + 8) * lda + k];
      }
#pragma unroll
      for (int ni = 0; ni < NI; ++ni) {
        int n = n0 + ni * 8 + 2 * t4;
        float b0 = B_KN ? B[(size_t)k * ldb + n] : B[(size_t)n * ldb + k];
        float b1 = B_KN ? B[(size_t)k * ldb + n + 1] : B[(size_t)(n + 1) * ldb + k];
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
          acc[mi][ni][0] = fmaf(a_lo[mi], b0, acc[mi][ni][0]);
          acc[mi][ni][1] = fmaf(a_lo[mi], b1, acc[mi][ni][1]);
          acc[mi][ni][2] = fmaf(a_hi[mi], b0, acc[mi][ni][2]);
          acc[mi][ni][3] = fmaf(a_hi[mi], b1, acc[mi][ni][3]);
        }
      }
    }
  }
};

// Tile product on fp32 shared-memory operands through the TF32 tensor-core path (m16n8k8): operands are expected
// to be rounded to TF32 already (to_tf32 when the tile is written), accumulation is fp32. Used where the operands of
// a 16-bit op have to carry more than 8 mantissa bits (differences of nearly cancelling sums downstream).
// Same conventions as WarpGemm: A_T / B_KN select the storage order, acc is the m16n8 fragment.
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
template <int MI, int NI, bool A_T, bool B_KN>
__device__ __forceinline__ void warp_gemm_tf32(float (&acc)[MI][NI][4], const float *A, int lda, int m0, const float *B, int ldb,
                                               int n0, int kdim) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  for (int k0 = 0; k0 < kdim; k0 += 8) {
    uint32_t af[MI][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi) {
      const int m = m0 + 16 * mi + g, k = k0 + t4;
      af[mi][0] = __float_as_uint(A_T ? A[k * lda + m] : A[m * lda + k]);
      af[mi][1] = __float_as_uint(A_T ? A[k * lda + m + 8] : A[(m + 8) * lda + k]);
      af[mi][2] = __float_as_uint(A_T ? A[(k + 4) * lda + m] : A[m * lda + k + 4]);
      af[mi][3] = __float_as_uint(A_T ? A[(k + 4) * lda + m + 8] : A[(m + 8) * lda + k + 4]);
    }
#pragma unroll
    for (int ni = 0; ni < NI; ++ni) {
      const int n = n0 + 8 * ni + g, k = k0 + t4;
      const uint32_t b0 = __float_as_uint(B_KN ? B[k * ldb + n] : B[n * ldb + k]);
      const uint32_t b1 = __float_as_uint(B_KN ? B[(k + 4) * ldb + n] : B[n * ldb + k + 4]);
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(acc[mi][ni][0]), "+f"(acc[mi][ni][1]), "+f"(acc[mi][ni][2]), "+f"(acc[mi][ni][3])
                     : "r"(af[mi][0]), "r"(af[mi][1]), "r"(af[mi][2]), "r"(af[mi][3]), "r"(b0), "r"(b1));
    }
  }
}
// fp32 operand tiles: true fp32 FMAs when the op's element type is fp32, the TF32 path for 16-bit element types
template <int MI, int NI, bool A_T, bool B_KN, typename T>
__device__ __forceinline__ void gemm_f32tile(float (&acc)[MI][NI][4], const float *A, int lda, int m0, const float *B, int ldb, int n0,
                                             int kdim) {
  if constexpr (sizeof(T) == 4) WarpGemm<MI, NI, A_T, B_KN, float>::run(acc, A, lda, m0, B, ldb, n0, kdim);
  else warp_gemm_tf32<MI, NI, A_T, B_KN>(acc, A, lda, m0, B, ldb, n0, kdim);
}
template <typename T> __device__ __forceinline__ float tile_round(float x) { return sizeof(T) == 4 ? x : to_tf32(x); }

// fp32 tile product with the contraction length known at compile time (fully unrolled, so the
// shared-memory operand loads of later steps overlap the FMAs of earlier ones)
template <int MI, int NI, int KD, bool A_T, bool B_KN>
__device__ __forceinline__ void warp_gemm_f32(float (&acc)[MI][NI][4], const float *A, int lda, int m0, const float *B, int ldb,
                                              int n0) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int k = 0; k < KD; ++k) {
    float a_lo[MI], a_hi[MI];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi) {
      const int m = m0 + mi * 16 + g;
      a_lo[mi] = A_T ? A[k * lda + m] : A[m * lda + k];
      a_hi[mi] = A_T ? A[k * lda + m + 8] : A[(m + 8) * lda + k];
    }
#pragma unroll
    for (int ni = 0; ni < NI; ++ni) {
      const int n = n0 + ni * 8 + 2 * t4;
      const float b0 = B_KN ? B[k * ldb + n] : B[n * ldb + k];
      const float b1 = B_KN ? B[k * ldb + n + 1] : B[(n + 1) * ldb + k];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi) {
        acc[mi][ni][0] = fmaf(a_lo[mi], b0, acc[mi][ni][0]);
        acc[mi][ni][1] = fmaf(a_lo[mi], b1, acc[mi][ni][1]);
        acc[mi][ni][2] = fmaf(a_hi[mi], b0, acc[mi][ni][2]);
        acc[mi][ni][3] = fmaf(a_hi[mi], b1, acc[mi][ni][3]);
      }
    }
  }
}

// dst[r][c] = T(src[r][c] * f[r]) over a [64 x cols] tile, 16 bytes per thread step (dst may equal src)
template <typename T>
__device__ __forceinline__ void tile_scale_rows(T *dst, const T *src, int ld, int cols, const float *f, int tid, int nthreads) {
  constexpr int EPV = 16 / sizeof(T);
  const int cpr = cols / EPV;
  for (int i = tid; i < C * cpr; i += nthreads) {
    const int r = i / cpr, c = (i - r * cpr) * EPV;
    int4 x = *reinterpret_cast<const int4 *>(src + r * ld + c);
    T *px = reinterpret_cast<T *>(&x);
    const float fr = f[r];
#pragma unroll
    for (int j = 0; j < EPV; ++j) px[j] = Num<T>::t(Num<T>::f(px[j]) * fr);
    *reinterpret_cast<int4 *>(dst + r * ld + c) = x;
  }
}

template <int MI, int NI> __device__ __forceinline__ void acc_zero(float (&acc)[MI][NI][4]) {
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int ni = 0; ni < NI; ++ni)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[mi][ni][r] = 0.f;
}

// store two adjacent accumulator columns as the element type
template <typename T> __device__ __forceinline__ void st_pair(T *p, float x, float y);
template <> __device__ __forceinline__ void st_pair<bf16>(bf16 *p, float x, float y) {
  *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(x, y);
}
template <> __device__ __forceinline__ void st_pair<__half>(__half *p, float x, float y) {
  *reinterpret_cast<__half2 *>(p) = __floats2half2_rn(x, y);
}
template <> __device__ __forceinline__ void st_pair<float>(float *p, float x, float y) {
  *reinterpret_cast<float2 *>(p) = make_float2(x, y);
}

// load two adjacent elements as floats
template <typename T> __device__ __forceinline__ float2 ld_pair(const T *p);
template <> __device__ __forceinline__ float2 ld_pair<bf16>(const bf16 *p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
}
template <> __device__ __forceinline__ float2 ld_pair<__half>(const __half *p) {
  return __half22float2(*reinterpret_cast<const __half2 *>(p));
}
template <> __device__ __forceinline__ float2 ld_pair<float>(const float *p) { return *reinterpret_cast<const float2 *>(p); }

// accumulator fragment -> shared tile (element type T), rows m0.., cols n0..
template <int MI, int NI, typename T>
__device__ __forceinline__ void acc_to_smem(const float (&acc)[MI][NI][4], T *s, int ld, int m0, int n0) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int ni = 0; ni < NI; ++ni) {
      int row = m0 + mi * 16 + g, col = n0 + ni * 8 + 2 * t4;
      st_pair<T>(s + (size_t)row * ld + col, acc[mi][ni][0], acc[mi][ni][1]);
      st_pair<T>(s + (size_t)(row + 8) * ld + col, acc[mi][ni][2], acc[mi][ni][3]);
    }
}

// helpers to walk an accumulator fragment with coordinates
#define FLAB_ACC_FOREACH(MI, NI, m0, n0, row, col, mi, ni, r)                         \
  _Pragma("unroll") for (int mi = 0; mi < (MI); ++mi)                                 \
  _Pragma("unroll") for (int ni = 0; ni < (NI); ++ni)                                 \
  _Pragma("unroll") for (int r = 0; r < 4; ++r)                                       \
    if (int row = (m0) + mi * 16 + ((threadIdx.x & 31) >> 2) + ((r >> 1) << 3); true) \
      if (int col = (n0) + ni * 8 + 2 * (threadIdx.x & 3) + (r & 1); true)

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
void set_error(const char *fmt, ...);
int check_launch(const char *what);

#define FLAB_REQUIRE(cond, code, ...) \
  do {                                \
    if (!(cond)) {                    \
      flab::set_error(__VA_ARGS__);   \
      return (code);                  \
    }                                 \
  } while (0)

#define FLAB_DISPATCH_16(dt, T, ...)                                              \
  switch (dt) {                                                                   \
    case FLAB_BF16: { using T = flab::bf16; __VA_ARGS__; } break;                 \
    case FLAB_FP16: { using T = __half; __VA_ARGS__; } break;                     \
    default: flab::set_error("dtype %d not supported by this entry point", (int)(dt)); return FLAB_E_UNSUPPORTED; \
  }
#define FLAB_DISPATCH_ALL(dt, T, ...)                                             \
  switch (dt) {                                                                   \
    case FLAB_BF16: { using T = flab::bf16; __VA_ARGS__; } break;                 \
    case FLAB_FP16: { using T = __half; __VA_ARGS__; } break;                     \
    case FLAB_FP32: { using T = float; __VA_ARGS__; } break;                      \
    default: flab::set_error("unknown dtype %d", (int)(dt)); return FLAB_E_BADARG; \
  }

template <typename KernelT> inline int set_smem(KernelT kernel, size_t bytes) {
  if (bytes > 227 * 1024) {
    set_error("kernel needs %zu bytes of shared memory (limit 232448)", bytes);
    return FLAB_E_UNSUPPORTED;
  }
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(%zu): %s", bytes, cudaGetErrorString(e));
      return FLAB_E_LAUNCH;
    }
  }
  return 0;
}

inline int check_common(const flab_args *a) {
  FLAB_REQUIRE(a != nullptr, FLAB_E_BADARG, "args is NULL");
  FLAB_REQUIRE(a->B > 0 && a->T > 0 && a->H > 0 && a->N > 0, FLAB_E_BADARG, "B,T,H,N must be positive (got %d,%d,%d,%d)",
               a->B, a->T, a->H, a->N);
  if (a->cu_seqlens) {
    FLAB_REQUIRE(a->B == 1 && !a->head_first, FLAB_E_BADARG, "variable-length input needs B == 1 and seq-first layout");
    FLAB_REQUIRE(a->chunk_indices && a->chunk_offsets, FLAB_E_BADARG, "variable-length input needs chunk_indices and chunk_offsets");
  } else {
    FLAB_REQUIRE(a->N == a->B, FLAB_E_BADARG, "fixed-length input needs N == B");
  }
  return 0;
}

}  // namespace flab
