// Host-side helpers shared by the C-ABI entry points: error reporting, argument
// checks and TMA tensor-map construction (driver entry point fetched through the
// runtime, so the library does not link libcuda directly).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

namespace semblo {

enum ReturnCode : int {
  SEMBLO_OK = 0,
  SEMBLO_EINVAL = -1,      // bad argument (shape, alignment, unsupported size)
  SEMBLO_ECUDA = -2,       // a CUDA runtime / driver call failed
  SEMBLO_ENOSPC = -3,      // caller-provided workspace too small
};

char* last_error_buffer();

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define SEMBLO_REQUIRE(cond, ...)                                        \
  do {                                                                   \
    if (!(cond)) return ::semblo::fail(::semblo::SEMBLO_EINVAL, __VA_ARGS__); \
  } while (0)

#define SEMBLO_CUDA(call)                                                           \
  do {                                                                              \
    cudaError_t e__ = (call);                                                       \
    if (e__ != cudaSuccess)                                                         \
      return ::semblo::fail(::semblo::SEMBLO_ECUDA, "%s failed: %s", #call,         \
                            cudaGetErrorString(e__));                               \
  } while (0)

#define SEMBLO_LAUNCH_CHECK()                                                       \
  do {                                                                              \
    cudaError_t e__ = cudaGetLastError();                                           \
    if (e__ != cudaSuccess)                                                         \
      return ::semblo::fail(::semblo::SEMBLO_ECUDA, "kernel launch failed at %s:%d: %s", \
                            __FILE__, __LINE__, cudaGetErrorString(e__));           \
  } while (0)

// bf16 tensor map with the 128-byte swizzle.  dims/strides innermost first; strides in
// bytes for dims 1.. (dim 0 is contiguous).  box[0] * 2 bytes must be 128.
int make_tensor_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box);

// Multiprocessors of the current device (148 if the query fails): persistent grids are sized by it.
int sm_count();

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace semblo
