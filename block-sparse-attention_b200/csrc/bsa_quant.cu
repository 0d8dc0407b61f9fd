// Sage FP8 quantiser (HBM-bound streaming): BF16 BHSD Q/K/V with D = 128 -> e4m3 bytes plus the
// multiplicative dequantisation scales.
//   Q: per token       scale = max(|row|, 1e-3) / 448, value = e4m3(bf16(q * bf16(1 / bf16(scale))))
//   K: per 16 tokens   over all 128 channels of the mean-centred K (mean over the sequence, per (b,h,c)),
//                      value = e4m3((k - mean) / scale); a zero-padded tail group is centred too
//   V: per (head, c)   scale = max(max_{b,s} |v|, 1e-3) / 448, value = e4m3(v * (1 / scale))
// Recipe of bsa_fp8_quant.py:10-104 (the Triton kernels behind quantize_sage_bhsd), pinned by
// tests/test_bsa_fp8_quant.py:34-63.
#include "bsa_b200.h"

#include <atomic>
#include "bsa_common.cuh"
#include "bsa_host.h"

namespace bsa {

constexpr int kStatChunk = 1024;  // tokens per statistics block

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}

// grid (chunks, B*H), 256 threads: thread t owns channels 8*(t%16)..+7 of token rows t/16, t/16+16, ...
__global__ void __launch_bounds__(256)
quant_stats_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                   float* __restrict__ ksum_part, float* __restrict__ vmax_part, int Sk, int chunks) {
  const int chunk = blockIdx.x;
  const long long bh = blockIdx.y;
  const int cg = threadIdx.x & 15;
  const int r0 = threadIdx.x >> 4;
  float ks[8], vm[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ks[i] = 0.f;
    vm[i] = 0.f;
  }
  const int s_begin = chunk * kStatChunk;
  const int s_end = min(Sk, s_begin + kStatChunk);
  for (int s = s_begin + r0; s < s_end; s += 16) {
    const long long off = (bh * Sk + s) * 128 + cg * 8;
    const uint4 kk = *reinterpret_cast<const uint4*>(k + off);
    const uint4 vv = *reinterpret_cast<const uint4*>(v + off);
    float kf[8], vf[8];
    unpack8(kk, kf);
    unpack8(vv, vf);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ks[i] += kf[i];
      vm[i] = fmaxf(vm[i], fabsf(vf[i]));
    }
  }
  __shared__ float s_k[16][128];
  __shared__ float s_v[16][128];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s_k[r0][cg * 8 + i] = ks[i];
    s_v[r0][cg * 8 + i] = vm[i];
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    float a = 0.f, m = 0.f;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      a += s_k[r][threadIdx.x];
      m = fmaxf(m, s_v[r][threadIdx.x]);
    }
    const long long o = (bh * chunks + chunk) * 128 + threadIdx.x;
    ksum_part[o] = a;
    vmax_part[o] = m;
  }
}

// grid (B*H), 128 threads: k_mean[b,h,c]; then v_scale[h,c] by blocks with b == 0 (needs all partials of
// every batch, which are complete because this is a separate launch)
__global__ void __launch_bounds__(128)
quant_finish_kernel(const float* __restrict__ ksum_part, const float* __restrict__ vmax_part,
                    float* __restrict__ k_mean, float* __restrict__ v_scale, int B, int H, int Sk, int chunks) {
  const int bh = blockIdx.x;
  const int c = threadIdx.x;
  float a = 0.f;
  for (int ch = 0; ch < chunks; ++ch) a += ksum_part[((long long)bh * chunks + ch) * 128 + c];
  k_mean[(long long)bh * 128 + c] = a / (float)Sk;
  if (bh < H) {
    const int h = bh;
    float m = 0.f;
    for (int b = 0; b < B; ++b)
      for (int ch = 0; ch < chunks; ++ch)
        m = fmaxf(m, vmax_part[(((long long)b * H + h) * chunks + ch) * 128 + c]);
    v_scale[h * 128 + c] = fmaxf(m, 1e-3f) / 448.0f;
  }
}

__device__ __forceinline__ uint2 to_e4m3x8(const float* f) {
  uint2 r;
  r.x = pack_e4m3x4(f[0], f[1], f[2], f[3]);
  r.y = pack_e4m3x4(f[4], f[5], f[6], f[7]);
  return r;
}

// grid (ceil(max(Sq,Sk)/128), B*H), 256 threads = 8 warps; a warp owns one 16-token group: lane l holds
// channels 8*(l%16)..+7 of token rows (l/16) + 2*j, j = 0..7.
__global__ void __launch_bounds__(256)
quant_apply_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                   const __nv_bfloat16* __restrict__ v, uint8_t* __restrict__ q8, uint8_t* __restrict__ k8,
                   uint8_t* __restrict__ v8, float* __restrict__ q_scale, float* __restrict__ k_scale,
                   const float* __restrict__ v_scale, const float* __restrict__ k_mean, int H, int Sq, int Sk) {
  const long long bh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = blockIdx.x * 8 + warp;  // 16-token group index
  const int s0 = group * 16;
  const int cg = lane & 15;
  const int rsub = lane >> 4;

  if (s0 < Sq) {
    uint4 raw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = s0 + rsub + 2 * j;
      raw[j] = (s < Sq) ? *reinterpret_cast<const uint4*>(q + (bh * Sq + s) * 128 + cg * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = s0 + rsub + 2 * j;
      float f[8];
      unpack8(raw[j], f);
      float am = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(f[i]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));  // 16-lane row
      const float scale = fmaxf(am, 1e-3f) / 448.0f;
      // BF16-rounded scale, reciprocal and product
      const float scale_bf = __bfloat162float(__float2bfloat16_rn(scale));
      const float rec_bf = __bfloat162float(__float2bfloat16_rn(1.0f / scale_bf));
      float g[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = __bfloat162float(__float2bfloat16_rn(f[i] * rec_bf));
      if (s < Sq) {
        *reinterpret_cast<uint2*>(q8 + (bh * Sq + s) * 128 + cg * 8) = to_e4m3x8(g);
        if (cg == 0) q_scale[bh * Sq + s] = scale;
      }
    }
  }

  if (s0 < Sk) {
    float mean[8], vrec[8];
    {
      const float4 m0 = *reinterpret_cast<const float4*>(k_mean + bh * 128 + cg * 8);
      const float4 m1 = *reinterpret_cast<const float4*>(k_mean + bh * 128 + cg * 8 + 4);
      mean[0] = m0.x; mean[1] = m0.y; mean[2] = m0.z; mean[3] = m0.w;
      mean[4] = m1.x; mean[5] = m1.y; mean[6] = m1.z; mean[7] = m1.w;
      const int h = (int)(bh % H);
#pragma unroll
      for (int i = 0; i < 8; ++i) vrec[i] = 1.0f / v_scale[h * 128 + cg * 8 + i];
    }
    uint4 kr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = s0 + rsub + 2 * j;
      kr[j] = (s < Sk) ? *reinterpret_cast<const uint4*>(k + (bh * Sk + s) * 128 + cg * 8) : make_uint4(0, 0, 0, 0);
    }
    // group absmax of the centred K; zero-padded tail rows are centred as well
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f[8];
      unpack8(kr[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(f[i] - mean[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float kscale = fmaxf(am, 1e-3f) / 448.0f;
    if (lane == 0) k_scale[bh * ((Sk + 15) / 16) + group] = kscale;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = s0 + rsub + 2 * j;
      if (s < Sk) {
        float f[8], g[8];
        unpack8(kr[j], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = __fdiv_rn(f[i] - mean[i], kscale);
        *reinterpret_cast<uint2*>(k8 + (bh * Sk + s) * 128 + cg * 8) = to_e4m3x8(g);
      }
    }
    uint4 vr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = s0 + rsub + 2 * j;
      vr[j] = (s < Sk) ? *reinterpret_cast<const uint4*>(v + (bh * Sk + s) * 128 + cg * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = s0 + rsub + 2 * j;
      if (s < Sk) {
        float f[8], g[8];
        unpack8(vr[j], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = f[i] * vrec[i];
        *reinterpret_cast<uint2*>(v8 + (bh * Sk + s) * 128 + cg * 8) = to_e4m3x8(g);
      }
    }
  }
}

}  // namespace bsa

using namespace bsa;

extern "C" int64_t bsa_quantize_sage_scratch_floats(int32_t B, int32_t H, int32_t Sk) {
  if (B < 1 || H < 1 || Sk < 1) return 0;
  const int64_t chunks = (Sk + kStatChunk - 1) / kStatChunk;
  return 2 * (int64_t)B * H * chunks * 128;
}

extern "C" int bsa_quantize_sage(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8,
                                 float* q_scale, float* k_scale, float* v_scale, float* k_mean, float* partials,
                                 int32_t B, int32_t H, int32_t Sq, int32_t Sk, void* cuda_stream) {
  if (!q || !k || !v || !q8 || !k8 || !v8 || !q_scale || !k_scale || !v_scale || !k_mean || !partials)
    return set_error(BSA_ERR_INVALID, "bsa_quantize_sage: null pointer");
  if (B < 1 || H < 1 || Sq < 1 || Sk < 1) return set_error(BSA_ERR_INVALID, "bsa_quantize_sage: non-positive extent");
  if ((long long)B * H > 65535) return set_error(BSA_ERR_UNSUPPORTED, "bsa_quantize_sage: B*H above 65535");
  {
    // the kernels read and write these tensors through 16-byte vector accesses
    const void* vec16[7] = {q, k, v, q8, k8, v8, k_mean};
    const char* names[7] = {"q", "k", "v", "q8", "k8", "v8", "k_mean"};
    for (int i = 0; i < 7; ++i)
      if ((reinterpret_cast<uintptr_t>(vec16[i]) & 15u) != 0)
        return set_error(BSA_ERR_INVALID, "bsa_quantize_sage: %s must be 16-byte aligned", names[i]);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int chunks = (Sk + kStatChunk - 1) / kStatChunk;
  float* ksum = partials;
  float* vmax = partials + (long long)B * H * chunks * 128;
  quant_stats_kernel<<<dim3(chunks, B * H), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(k),
                                                          reinterpret_cast<const __nv_bfloat16*>(v), ksum, vmax, Sk,
                                                          chunks);
  quant_finish_kernel<<<B * H, 128, 0, st>>>(ksum, vmax, k_mean, v_scale, B, H, Sk, chunks);
  const int smax = Sq > Sk ? Sq : Sk;
  quant_apply_kernel<<<dim3((smax + 127) / 128, B * H), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k),
      reinterpret_cast<const __nv_bfloat16*>(v), reinterpret_cast<uint8_t*>(q8), reinterpret_cast<uint8_t*>(k8),
      reinterpret_cast<uint8_t*>(v8), q_scale, k_scale, v_scale, k_mean, H, Sq, Sk);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "quantiser launch: %s", cudaGetErrorString(e));
  return BSA_OK;
}

// -------------------------------------------------------------------------------------------------
// Quantiser entry point that owns its scratch (no counterpart in the reference).
//
// Some hosts of this library have no way to hand over scratch memory: an inference server that froze
// its memory pool after start-up, a C or Rust service that links the library without any tensor
// allocator, a latency-critical loop where a cudaMalloc would stall the whole device.  For them the
// K-mean vector and the per-chunk statistics live in the fixed device array below instead of in
// caller-provided buffers.  The array is part of the library image: every GPU that loads the library
// holds these 4 MiB until the process exits.
// -------------------------------------------------------------------------------------------------
namespace bsa {
constexpr long long kStaticScratchFloats = BSA_QUANTIZE_STATIC_SCRATCH_FLOATS;  // 4 MiB
static __device__ __align__(256) float g_quant_scratch[kStaticScratchFloats];
}  // namespace bsa

extern "C" int bsa_quantize_sage_static(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8,
                                        float* q_scale, float* k_scale, float* v_scale, int32_t B, int32_t H,
                                        int32_t Sq, int32_t Sk, void* cuda_stream) {
  if (B < 1 || H < 1 || Sq < 1 || Sk < 1)
    return set_error(BSA_ERR_INVALID, "bsa_quantize_sage_static: non-positive extent");
  const long long mean_floats = (long long)B * H * 128;
  const long long need = mean_floats + bsa_quantize_sage_scratch_floats(B, H, Sk);
  if (need > kStaticScratchFloats)
    return set_error(BSA_ERR_WORKSPACE,
                     "bsa_quantize_sage_static: B*H*(1 + 2*ceil(Sk/1024))*128 = %lld floats exceed the built-in "
                     "scratch of %lld floats; use bsa_quantize_sage with caller-provided scratch",
                     need, kStaticScratchFloats);
  // In host code the array's name is only a handle; the device address has to be asked for, once per
  // device, with that device current.  This first call per device is the set-up.
  // (atomic slots: two host threads making the first call on one device both look the address up and store the
  // same value)
  static std::atomic<float*> scratch_of_device[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return set_error(BSA_ERR_CUDA, "bsa_quantize_sage_static: cannot identify the current device");
  float* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    void* addr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&addr, g_quant_scratch);
    if (e != cudaSuccess || addr == nullptr)
      return set_error(BSA_ERR_CUDA, "bsa_quantize_sage_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    scratch = static_cast<float*>(addr);
    scratch_of_device[dev].store(scratch, std::memory_order_release);
  }
  // Every slot that is read has been written earlier in the same call (statistics kernel -> finish kernel
  // -> apply kernel), so nothing has to be cleared between calls.
  return bsa_quantize_sage(q, k, v, q8, k8, v8, q_scale, k_scale, v_scale, /*k_mean=*/scratch,
                           /*partials=*/scratch + mean_floats, B, H, Sq, Sk, cuda_stream);
}
