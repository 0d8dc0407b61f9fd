// Host-side helpers of libbsa_b200.so: error text, tensor-map encoding, device queries.
#include "bsa_host.h"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "bsa_b200.h"
#include "bsa_common.cuh"

namespace bsa {

// Self-test of the bounded wait: two warps wait on an mbarrier that nobody ever arrives at.  The first thread
// whose budget runs out records the status word and raises the abort flag, the other warp leaves through the
// flag, and both fall through to the end of the kernel - the same path every role of the tcgen05 kernels takes.
__global__ void __launch_bounds__(64, 1) selftest_wait_kernel(int* status, int* returned, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  __syncthreads();
  WaitCtx ctx{&abort_flag, status};
  const bool ok = mbar_wait_limit(smem_u32(&bar), 0, ctx, 900 + (int)(threadIdx.x >> 5), limit_ns);
  __syncthreads();  // the common teardown point
  if (threadIdx.x == 0) *returned = ok ? 2 : 1;
}

static thread_local char g_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_error(BSA_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return set_error(BSA_ERR_INVALID, "%s: base address must be 16-byte aligned", what);
  cuuint64_t gdims[5];
  cuuint64_t gstr[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    if (strides_bytes[i] % 16 != 0 || strides_bytes[i] == 0 || strides_bytes[i] >= (1ull << 40))
      return set_error(BSA_ERR_INVALID, "%s: stride %d (%llu bytes) must be a non-zero multiple of 16 below 2^40",
                       what, i + 1, (unsigned long long)strides_bytes[i]);
    gstr[i] = strides_bytes[i];
  }
  CUresult r = fn(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstr, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(BSA_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return 0;
}

}  // namespace bsa

extern "C" int bsa_abi_version(void) { return BSA_B200_ABI_VERSION; }

extern "C" const char* bsa_last_error(void) { return bsa::g_error; }

extern "C" int bsa_selftest_wait(uint64_t limit_ns, int32_t* status, int32_t* returned, void* cuda_stream) {
  if (!status || !returned) return bsa::set_error(BSA_ERR_INVALID, "bsa_selftest_wait: null pointer");
  if (limit_ns == 0 || limit_ns > 1000000000ull)
    return bsa::set_error(BSA_ERR_INVALID, "bsa_selftest_wait: limit must be in (0, 1 s]");
  bsa::selftest_wait_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(status, returned, limit_ns);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return bsa::set_error(BSA_ERR_CUDA, "selftest launch: %s", cudaGetErrorString(e));
  return BSA_OK;
}

extern "C" int bsa_num_sms(int device) {
  static int cached[64];
  if (device < 0 || device >= 64) return -1;
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    cached[device] = n;
  }
  return cached[device];
}
