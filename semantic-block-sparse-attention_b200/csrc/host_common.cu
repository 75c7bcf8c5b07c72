#include "host_common.h"

#include "../../include/semblo_b200.h"

namespace semblo {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int sm_count() {
  static thread_local int cached_device = -1, cached = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_device) {
    int n = 0;
    cached = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0 ? n : 148;
    cached_device = dev;
  }
  return cached;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

int make_tensor_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(SEMBLO_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if (reinterpret_cast<uintptr_t>(base) & 15)
    return fail(SEMBLO_EINVAL, "tensor base %p is not 16-byte aligned", base);
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      if (strides_bytes[i - 1] & 15)
        return fail(SEMBLO_EINVAL, "tensor stride %llu is not a multiple of 16 bytes",
                    (unsigned long long)strides_bytes[i - 1]);
      gstrides[i - 1] = strides_bytes[i - 1];
    }
  }
  if (box[0] * 2 != 128) return fail(SEMBLO_EINVAL, "inner box must span 128 bytes");
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdims,
                  gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SEMBLO_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return SEMBLO_OK;
}

}  // namespace semblo

extern "C" int semblo_version(void) { return 100; }

extern "C" const char* semblo_last_error(void) { return semblo::last_error_buffer(); }
