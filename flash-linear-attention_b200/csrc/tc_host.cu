// Host-side TMA tensor-map construction.  cuTensorMapEncodeTiled is fetched through the runtime's
// driver entry point query, so the library has no link-time dependency on libcuda and still loads on
// a machine without a driver (where only the CPU-side tests run).
#include "tc.cuh"

namespace flab {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rank <= 4; dims[0] is the contiguous extent; strides_bytes[i] is the stride of dims[i+1].
// 128-byte swizzle, zero fill outside the tensor.
int make_tensor_map_bf16(CUtensorMap *map, const void *base, int rank, const uint64_t *dims, const uint64_t *strides_bytes,
                         const uint32_t *box, int elem_fp16) {
  EncodeTiledFn fn = encode_fn();
  // A driver-API call needs a current context; a thread that has only used the runtime lazily (an
  // autograd worker thread, say) may not have bound the primary context yet.  cudaSetDevice binds it
  // without touching the allocator, so this is legal while a stream is being captured.
  static thread_local bool bound = false;
  if (!bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
    bound = true;
  }
  FLAB_REQUIRE(fn != nullptr, FLAB_E_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[4];
  cuuint64_t gstr[4];
  cuuint32_t bx[4], es[4];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = fn(map, elem_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank,
                  const_cast<void *>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FLAB_REQUIRE(r == CUDA_SUCCESS, FLAB_E_BADARG, "cuTensorMapEncodeTiled failed with code %d (base %p must be 16-byte aligned, strides multiples of 16)",
               (int)r, base);
  return 0;
}


int make_token_map(CUtensorMap *map, const void *base, const flab_args *a, int D) {
  const uint64_t e = 2;
  if (!a->head_first) {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)a->H, (uint64_t)a->T, (uint64_t)a->B};
    const uint64_t str[3] = {(uint64_t)D * e, (uint64_t)a->H * D * e, (uint64_t)a->T * a->H * D * e};
    const uint32_t box[4] = {64, 1, 64, 1};
    return make_tensor_map_bf16(map, base, 4, dims, str, box, a->dtype == FLAB_FP16);
  }
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)a->T, (uint64_t)a->H, (uint64_t)a->B};
  const uint64_t str[3] = {(uint64_t)D * e, (uint64_t)a->T * D * e, (uint64_t)a->H * a->T * D * e};
  const uint32_t box[4] = {64, 64, 1, 1};
  return make_tensor_map_bf16(map, base, 4, dims, str, box, a->dtype == FLAB_FP16);
}

int make_state_map(CUtensorMap *map, const void *base, const flab_args *a, int box_rows) {
  const uint64_t dims[2] = {(uint64_t)a->V, (uint64_t)a->NT * a->H * a->K};
  const uint64_t str[1] = {(uint64_t)a->V * 2};
  const uint32_t box[2] = {64, (uint32_t)box_rows};
  return make_tensor_map_bf16(map, base, 2, dims, str, box, a->dtype == FLAB_FP16);
}

#define FLAB_ERROR_UNITS(X) X(tc_chunk_o_error) X(recurrent_error) X(tc_delta_h_error) X(tc_dqkwg_error) X(tc_wy_bwd_error) X(tc_wy_fwd_error) X(tc_selftest_error)
#define FLAB_DECLARE_UNIT(name) \
  int name();                   \
  int name##_clear();
FLAB_ERROR_UNITS(FLAB_DECLARE_UNIT)

}  // namespace flab

extern "C" int flab_tc_error_state(void) {
  int e = 0;
#define FLAB_READ_UNIT(name) \
  if (!e) e = flab::name();
  FLAB_ERROR_UNITS(FLAB_READ_UNIT)
  return e;
}

extern "C" int flab_tc_error_clear(void) {
  int e = 0;
#define FLAB_CLEAR_UNIT(name) e |= flab::name##_clear();
  FLAB_ERROR_UNITS(FLAB_CLEAR_UNIT)
  return e ? FLAB_E_LAUNCH : FLAB_OK;
}

extern "C" int flab_tc_check(void) {
  const int e = flab_tc_error_state();
  if (e == 0) return FLAB_OK;
  flab::set_error("a bounded device-side wait ran out (wait id %d): the results of the kernels launched since the last check are invalid", e);
  return FLAB_E_TIMEOUT;
}
