// Top-k block selection: the step that produces the q2k index (pooled block scores -> the k best KV
// blocks of every query block, ids ascending).  Integer/HBM-bound work, deterministic.
//
// The reference describes the step only through its benchmark recipe (tests/bench_cutedsl_performance.py:
// 131-167: pooled scores -> torch.topk(sorted=False) -> ascending sort -> int32) and in prose
// (design/fp8/results.md:635-636: mean-pool, top-k, complete K-block index layout).  Three kernels:
//   block_mean:   x [B,H,S,D] bf16 -> per-block mean [B,H,N,D] fp32      (reads x once)
//   pooled_score: qm [.,Nq,D], km [.,Nkv,D] -> scores [.,Nq,Nkv] fp32    (fixed summation order)
//   topk_rows:    scores [rows,Nkv] -> index [rows,cap], first k entries (bitonic sorts in shared memory)
#include "bsa_b200.h"
#include "bsa_common.cuh"
#include "bsa_host.h"

#include <cuda_bf16.h>

namespace bsa {

// ------------------------------------------------------------------------------------------------
// per-block mean: one warp per (b, h, block); lanes stride over the channels, 4 per load
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
block_mean_kernel(const __nv_bfloat16* __restrict__ x, long long sb, long long sh, long long ss, int H, int S, int D,
                  int blk, int N, long long rows, float* __restrict__ out) {
  const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int n = (int)(r % N);
  const long long bh = r / N;
  const int h = (int)(bh % H);
  const long long b = bh / H;
  const int t0 = n * blk;
  const int cnt = min(blk, S - t0);
  const __nv_bfloat16* base = x + b * sb + h * sh + (long long)t0 * ss;
  for (int c = lane * 4; c < D; c += 128) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int t = 0; t < cnt; ++t) {
      const uint2 v = *reinterpret_cast<const uint2*>(base + (long long)t * ss + c);
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
      a0 += lo.x;
      a1 += lo.y;
      a2 += hi.x;
      a3 += hi.y;
    }
    const float inv = cnt > 0 ? 1.f / (float)cnt : 0.f;
    *reinterpret_cast<float4*>(out + r * D + c) = make_float4(a0 * inv, a1 * inv, a2 * inv, a3 * inv);
  }
}

// ------------------------------------------------------------------------------------------------
// pooled scores: 16 x 16 output tile per CTA, channels staged through shared memory 32 at a time;
// every output is one thread's sum over d = 0, 1, 2, ... (fixed order)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
pooled_score_kernel(const float* __restrict__ qm, const float* __restrict__ km, int Nq, int Nkv, int D, float scale,
                    float* __restrict__ scores) {
  __shared__ float sq[16][33], sk[16][33];
  const int bh = blockIdx.z;
  const int m0 = blockIdx.y * 16, j0 = blockIdx.x * 16;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const float* q = qm + (long long)bh * Nq * D;
  const float* k = km + (long long)bh * Nkv * D;
  float acc = 0.f;
  for (int d0 = 0; d0 < D; d0 += 32) {
    for (int e = threadIdx.x; e < 16 * 32; e += 256) {
      const int rr = e >> 5, dd = e & 31;
      sq[rr][dd] = (m0 + rr < Nq && d0 + dd < D) ? q[(long long)(m0 + rr) * D + d0 + dd] : 0.f;
      sk[rr][dd] = (j0 + rr < Nkv && d0 + dd < D) ? k[(long long)(j0 + rr) * D + d0 + dd] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int dd = 0; dd < 32; ++dd) acc = fmaf(sq[ty][dd], sk[tx][dd], acc);
    __syncthreads();
  }
  if (m0 + ty < Nq && j0 + tx < Nkv) scores[((long long)bh * Nq + m0 + ty) * Nkv + j0 + tx] = acc * scale;
}

// ------------------------------------------------------------------------------------------------
// top-k of one row per CTA.  Keys are (orderable score << 32) | ~id, so a descending sort puts higher
// scores first and, among equal scores, lower ids first; the k winning ids are then sorted ascending.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t orderable(float f) {
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;  // NaN of either sign ranks above +inf (torch.topk)
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T, bool DESC>
__device__ __forceinline__ void bitonic_sort_shared(T* a, int n_pow2) {
  for (int size = 2; size <= n_pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int t = threadIdx.x; t < (n_pow2 >> 1); t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool up = ((lo & size) == 0) != DESC;  // ascending run?
        const T x = a[lo], y = a[hi];
        if ((x > y) == up) {
          a[lo] = y;
          a[hi] = x;
        }
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(1024)
topk_rows_kernel(const float* __restrict__ scores, int Nkv, int n_pow2, int k, int k_pow2, int cap,
                 int32_t* __restrict__ index) {
  extern __shared__ __align__(16) unsigned long long keys[];  // n_pow2 keys; the ids reuse the front
  const long long row = blockIdx.x;
  const float* srow = scores + row * Nkv;
  for (int i = threadIdx.x; i < n_pow2; i += blockDim.x) {
    keys[i] = (i < Nkv) ? (((unsigned long long)orderable(srow[i]) << 32) | (unsigned long long)(~(uint32_t)i)) : 0ull;
  }
  bitonic_sort_shared<unsigned long long, true>(keys, n_pow2);
  // winners -> ids (registers first: the id array aliases the key array)
  uint32_t* ids = reinterpret_cast<uint32_t*>(keys);
  uint32_t mine[4];  // k_pow2 <= 4 * blockDim.x is guaranteed by the host
  int cnt = 0;
  for (int i = threadIdx.x; i < k_pow2; i += blockDim.x) mine[cnt++] = (i < k) ? ~(uint32_t)(keys[i] & 0xffffffffull) : 0x7fffffffu;
  __syncthreads();
  cnt = 0;
  for (int i = threadIdx.x; i < k_pow2; i += blockDim.x) ids[i] = mine[cnt++];
  bitonic_sort_shared<uint32_t, false>(ids, k_pow2);
  for (int i = threadIdx.x; i < k; i += blockDim.x) index[row * cap + i] = (int32_t)ids[i];
}

}  // namespace bsa

using namespace bsa;

static int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

extern "C" int bsa_block_mean(const void* x, const int64_t* stride, int32_t B, int32_t H, int32_t S, int32_t D,
                              int32_t blk, float* out, void* cuda_stream) {
  if (!x || !stride || !out) return set_error(BSA_ERR_INVALID, "bsa_block_mean: null pointer");
  if (B < 1 || H < 1 || S < 1 || D < 4 || D % 4 != 0 || blk < 1)
    return set_error(BSA_ERR_INVALID, "bsa_block_mean: bad extents (D must be a positive multiple of 4)");
  if ((stride[0] | stride[1] | stride[2]) % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 7u) != 0)
    return set_error(BSA_ERR_INVALID, "bsa_block_mean: strides must be multiples of 4 elements, base 8-byte aligned");
  const int N = (S + blk - 1) / blk;
  const long long rows = (long long)B * H * N;
  block_mean_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), stride[0], stride[1], stride[2], H, S, D, blk, N, rows, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_block_mean launch: %s", cudaGetErrorString(e));
  return BSA_OK;
}

extern "C" int bsa_pooled_scores(const float* qm, const float* km, int32_t BH, int32_t Nq, int32_t Nkv, int32_t D,
                                 float scale, float* scores, void* cuda_stream) {
  if (!qm || !km || !scores) return set_error(BSA_ERR_INVALID, "bsa_pooled_scores: null pointer");
  if (BH < 1 || Nq < 1 || Nkv < 1 || D < 1 || BH > 65535)
    return set_error(BSA_ERR_INVALID, "bsa_pooled_scores: bad extents (batch*heads <= 65535)");
  dim3 grid((unsigned)((Nkv + 15) / 16), (unsigned)((Nq + 15) / 16), (unsigned)BH);
  if (grid.y > 65535) return set_error(BSA_ERR_UNSUPPORTED, "bsa_pooled_scores: too many query blocks");
  pooled_score_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(qm, km, Nq, Nkv, D, scale, scores);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_pooled_scores launch: %s", cudaGetErrorString(e));
  return BSA_OK;
}

extern "C" int bsa_topk_q2k(const float* scores, int64_t rows, int32_t Nkv, int32_t k, int32_t cap, int32_t* index,
                            void* cuda_stream) {
  if (!scores || !index) return set_error(BSA_ERR_INVALID, "bsa_topk_q2k: null pointer");
  if (rows < 0 || Nkv < 1 || k < 1 || k > Nkv || cap < k) return set_error(BSA_ERR_INVALID, "bsa_topk_q2k: need 1 <= k <= Nkv, cap >= k");
  if (Nkv > BSA_TOPK_MAX_BLOCKS) return set_error(BSA_ERR_UNSUPPORTED, "bsa_topk_q2k: at most %d KV blocks per row", BSA_TOPK_MAX_BLOCKS);
  if (rows > 0x7fffffffLL) return set_error(BSA_ERR_UNSUPPORTED, "bsa_topk_q2k: too many rows");
  if (rows == 0) return BSA_OK;
  const int n_pow2 = next_pow2(Nkv), k_pow2 = next_pow2(k);
  const int threads = 256;
  if (k_pow2 > 4096) return set_error(BSA_ERR_UNSUPPORTED, "bsa_topk_q2k: at most 4096 blocks can be selected per row");
  const size_t smem = (size_t)n_pow2 * sizeof(unsigned long long);
  cudaError_t e = cudaFuncSetAttribute(topk_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_topk_q2k: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  // a thread keeps at most 4 winners in registers between the two sorts: use enough threads for k
  const int t = k_pow2 > 4 * threads ? 1024 : threads;
  topk_rows_kernel<<<(unsigned)rows, t, smem, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(scores, Nkv, n_pow2, k, k_pow2,
                                                                                           cap, index);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_topk_q2k launch: %s", cudaGetErrorString(e));
  return BSA_OK;
}
