// Split-KV combine: LSE-weighted merge of FP32 partial outputs into the BF16 output.
//   lse = log sum_s exp(lse_s),   out = sum_s exp(lse_s - lse) * O_s
// One warp per query row (D = 128: one float4 per lane); pure HBM streaming, no shared memory.
// Semantics of csrc/fwd/sm100_blk64/bsa_fwd_combine.py:253-566 (rows whose partial LSEs are all -inf
// give zeros and lse = -inf, :458-468).
#include "bsa_b200.h"
#include "bsa_common.cuh"
#include "bsa_host.h"

namespace bsa {

constexpr int kCombineWarps = 8;

__global__ void __launch_bounds__(kCombineWarps * 32)
bsa_combine_kernel(const float* __restrict__ po, const float* __restrict__ plse,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int splits, long long rows,
                   int H, int Sq, long long os_b, long long os_h, long long os_s) {
  const long long row = (long long)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;

  // pass 1: max and sum of exp over the splits (lanes stride over splits)
  float m = -INFINITY;
  for (int s = lane; s < splits; s += 32) m = fmaxf(m, plse[(long long)s * rows + row]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.f;
  if (m != -INFINITY) {
    for (int s = lane; s < splits; s += 32) sum += __expf(plse[(long long)s * rows + row] - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float lse_all = (m == -INFINITY) ? -INFINITY : (m + __logf(sum));
  const float inv = (sum > 0.f) ? 1.f / sum : 0.f;

  // pass 2: weighted sum of the partial rows
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* src = reinterpret_cast<const float4*>(po) + row * 32 + lane;
  const long long split_stride4 = rows * 32;
  int s = 0;
  for (; s + 4 <= splits; s += 4) {
    float w[4];
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float l = plse[(long long)(s + u) * rows + row];
      w[u] = (l == -INFINITY) ? 0.f : __expf(l - m) * inv;
      v[u] = __ldcs(src + (long long)(s + u) * split_stride4);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (w[u] != 0.f) {  // an empty split may hold anything finite; skip it exactly
        acc.x = fmaf(w[u], v[u].x, acc.x);
        acc.y = fmaf(w[u], v[u].y, acc.y);
        acc.z = fmaf(w[u], v[u].z, acc.z);
        acc.w = fmaf(w[u], v[u].w, acc.w);
      }
    }
  }
  for (; s < splits; ++s) {
    const float l = plse[(long long)s * rows + row];
    const float w = (l == -INFINITY) ? 0.f : __expf(l - m) * inv;
    const float4 v = __ldcs(src + (long long)s * split_stride4);
    if (w != 0.f) {
      acc.x = fmaf(w, v.x, acc.x);
      acc.y = fmaf(w, v.y, acc.y);
      acc.z = fmaf(w, v.z, acc.z);
      acc.w = fmaf(w, v.w, acc.w);
    }
  }
  const int sq = (int)(row % Sq);
  const long long bh = row / Sq;
  const int h = (int)(bh % H);
  const long long b = bh / H;
  __nv_bfloat16* dst = out + b * os_b + h * os_h + (long long)sq * os_s + lane * 4;
  uint2 packed;
  packed.x = pack_bf16x2(acc.x, acc.y);
  packed.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(dst) = packed;
  if (lse != nullptr && lane == 0) lse[row] = lse_all;
}

}  // namespace bsa

using namespace bsa;

extern "C" int bsa_fwd_combine(const float* partial_o, const float* partial_lse, void* out, float* lse,
                               int32_t splits, int32_t B, int32_t H, int32_t Sq, int32_t D,
                               const int64_t o_stride[3], void* cuda_stream) {
  if (!partial_o || !partial_lse || !out || !o_stride) return set_error(BSA_ERR_INVALID, "bsa_fwd_combine: null pointer");
  if (D != 128) return set_error(BSA_ERR_UNSUPPORTED, "bsa_fwd_combine: D must be 128");
  if (splits < 1 || B < 1 || H < 1 || Sq < 1) return set_error(BSA_ERR_INVALID, "bsa_fwd_combine: non-positive extent");
  if ((o_stride[0] | o_stride[1] | o_stride[2]) % 4 != 0 || (reinterpret_cast<uintptr_t>(out) & 7))
    return set_error(BSA_ERR_INVALID, "bsa_fwd_combine: output rows must be 8-byte aligned");
  const long long rows = (long long)B * H * Sq;
  const long long blocks = (rows + kCombineWarps - 1) / kCombineWarps;
  if (blocks > 0x7fffffffLL) return set_error(BSA_ERR_UNSUPPORTED, "bsa_fwd_combine: too many rows");
  bsa_combine_kernel<<<(unsigned)blocks, kCombineWarps * 32, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(
      partial_o, partial_lse, reinterpret_cast<__nv_bfloat16*>(out), lse, splits, rows, H, Sq, o_stride[0],
      o_stride[1], o_stride[2]);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "combine launch: %s", cudaGetErrorString(e));
  return BSA_OK;
}
