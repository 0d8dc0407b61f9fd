// Block-sparse attention backward for sm_100a (BF16, MHA, D = 128, 128-token blocks).
//
// Three launches, no atomics anywhere, every accumulation in a fixed order (bit-reproducible):
//   1. preprocess : delta[row] = -sum_d O*dO, lse_log2[row] = -lse*log2(e), both stored NEGATED so that the main
//                   kernels add them with packed fp32x2 instructions (-inf for empty rows so that
//                   the recomputed probabilities are exactly 0), both padded to whole 128-row tiles
//   2. dQ kernel  : one work item per query tile, driven by the q2k index.  Per selected KV block:
//                   S = Q K^T, dP = dO V^T, P = exp2(S*scale - lse), dS = P o (dP - delta) (bf16, back to
//                   tensor memory), dQ += dS K.  dQ stays in tensor memory for the whole tile.
//   3. dK/dV kernel: one work item per KV block, driven by the k2q CSR (all query groups of the block
//                   are walked by the same CTA, so nothing has to be reduced across CTAs).  Per query
//                   tile of the CSR row: S^T = K Q^T, dP^T = V dO^T, P^T and dS^T (bf16) go back to
//                   tensor memory and feed dV += P^T dO and dK += dS^T Q.
// The probabilities are recomputed in both kernels (7 GEMMs per active pair instead of the 5 of a fused
// kernel); in exchange dQ needs no FP32 workspace, no reduce-add traffic and no post-processing pass.
//
// Math and rounding points follow the reference csrc/bwd/sm100_blk128/bsa_bwd_sm100.py (P and dS rounded
// to bf16 before the dV/dK/dQ GEMMs :1766, :1808-1809; dK and dQ scaled by softmax_scale at the end
// :1864, :2351), its preprocess csrc/bwd/bsa_bwd_preprocess.py:184-324 and its CSR walk :86-112.
//
// Warp roles: warps 0-7 compute in both kernels (two groups of 128 threads, thread = tensor-memory lane, group g
// owns columns [64g, 64g+64) of the score tiles).  dQ kernel (384 threads): warps 8, 9 and 10 issue the MMAs of
// one dependency chain each (S, dQ, dP), warp 11 is the TMA producer.  dK/dV kernel (352 threads): warps 8 and 9
// issue MMAs, warp 10 is the TMA producer.
#include "bsa_b200.h"
#include "bsa_common.cuh"
#include "bsa_host.h"

#ifdef BSA_PHASE_TIMERS
// Development builds only (build.py --phase-timers): per-role clock counters, read by bsa_bwd_phase_timers().
__device__ unsigned long long g_bwd_phase[128];
#define PTB_FLUSH(base) PT_FLUSH_TO(g_bwd_phase, base)
#else
#define PTB_FLUSH(base)
#endif

namespace bsa {

constexpr int kBwdMmaWarp = 8;
constexpr int kDqThreads = 384;  // dQ kernel: warps 8, 9 and 10 issue MMAs, warp 11 loads
constexpr int kDqLoadWarp = 11;
constexpr int kDkvThreads = 352;  // dK/dV kernel: warps 8 and 9 issue MMAs, warp 10 loads
constexpr int kDkvLoadWarp = 10;
// Work item of this CTA in band `band`.  Natural order: CTA c takes c, G + c, 2G + c, ...  With a (longest-first)
// order list the bands are walked back and forth (c, 2G-1-c, 2G+c, ...), so that every CTA gets a similar total.
// Returns -1 when the band holds no item for this CTA.
__device__ __forceinline__ int bwd_work_at(const int32_t* order, int band, int num_work, int* status) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  const int wi = band * G + ((order != nullptr && (band & 1)) ? (G - 1 - c) : c);
  if (wi >= num_work) return -1;
  if (order == nullptr) return wi;
  int w = order[wi];
  if (w < 0 || w >= num_work) {  // a corrupt order must not turn into a wild access
    if (atomicCAS(status, 0, (int)kStatusBadIndex) == 0) status[2] = w;
    w = 0;
  }
  return w;
}

constexpr int kTile = 128 * 128 * 2;  // bytes of one bf16 128x128 tile
constexpr int kSlab = 128 * 128;      // bytes of one 64-column slab

struct BwdParams {
  const int32_t* __restrict__ q2k_index;
  const int32_t* __restrict__ q2k_nums;
  const int32_t* __restrict__ csr_offsets;
  const int32_t* __restrict__ csr_indices;
  const int32_t* __restrict__ order_q;      // optional work orders (longest first) of the two main kernels
  const int32_t* __restrict__ order_kv;
  const int32_t* __restrict__ block_sizes;  // optional valid-token counts of the KV blocks
  long long bs_stride_b, bs_stride_h;
  const float* __restrict__ lse_log2;  // [B,H,Nq*128]  -lse * log2(e)
  const float* __restrict__ delta;     // [B,H,Nq*128]  -sum_d O dO
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int* status;
  long long dq_stride[3], dk_stride[3], dv_stride[3];
  long long idx_cap;  // entries per (b,h) of csr_indices
  int fixed_count, cap;
  int B, H, Sq, Sk, Nq, Nkv, G;
  int D;  // head dimension (64 or 128): a 64-wide head rides on the 128-wide tiles, the tensor maps zero-fill
  float scale_log2, softmax_scale;
};

// ------------------------------------------------------------------------------------------------
// 1. preprocess
// ------------------------------------------------------------------------------------------------
// HBM-bound: reads O and dO once.  A warp handles eight consecutive padded rows: sixteen lanes per row with
// 16 bytes each, all eight loads of a thread in flight before the first use.
constexpr int kPreRowsPerWarp = 8;
__global__ void __launch_bounds__(256)
bwd_preprocess_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                      const float* __restrict__ lse, float* __restrict__ lse_log2, float* __restrict__ delta,
                      long long os_b, long long os_h, long long os_s, long long ds_b, long long ds_h, long long ds_s,
                      int H, int Sq, int SqPad, long long rows_pad, int D) {
  const long long row0 = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * kPreRowsPerWarp;
  if (row0 >= rows_pad) return;
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 4, chunk = lane & 15;  // two rows per pass, sixteen 16-byte chunks per row
  // the eight rows of a warp lie in one (batch, head) plane: the padded length is a multiple of 64
  const long long bh = row0 / SqPad;
  const int s0 = (int)(row0 - bh * SqPad);
  const int h = (int)(bh % H);
  const long long b = bh / H;
  const __nv_bfloat16* o_base = o + b * os_b + h * os_h + chunk * 8;
  const __nv_bfloat16* d_base = d_o + b * ds_b + h * ds_h + chunk * 8;
  uint4 ov[4], dv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int s = s0 + 2 * i + sub;
    ov[i] = make_uint4(0, 0, 0, 0);
    dv[i] = make_uint4(0, 0, 0, 0);
    if (s < Sq && chunk * 8 < D) {
      ov[i] = *reinterpret_cast<const uint4*>(o_base + (long long)s * os_s);
      dv[i] = *reinterpret_cast<const uint4*>(d_base + (long long)s * ds_s);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int s = s0 + 2 * i + sub;
    const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov[i]);
    const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv[i]);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(o2[e]);
      const float2 c = __bfloat1622float2(d2[e]);
      acc = fmaf(a.x, c.x, acc);
      acc = fmaf(a.y, c.y, acc);
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);  // within the half warp
    if (chunk == 0) {
      float l = INFINITY;
      if (s < Sq) {
        const float lv = lse[bh * Sq + s];
        l = (lv == -INFINITY) ? INFINITY : lv * kLog2e;
      }
      delta[bh * SqPad + s] = -acc;
      lse_log2[bh * SqPad + s] = -l;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// shared pieces of the two main kernels
// ------------------------------------------------------------------------------------------------
// Valid tokens of KV block j of (b, h): min(block_sizes[j], tokens physically left), 0 for ids out of range.
template <int BLK>
__device__ __forceinline__ int bwd_block_len(const BwdParams& p, int b, int h, int j) {
  if (j < 0 || j >= p.Nkv) return 0;
  int lim = min(BLK, p.Sk - j * BLK);
  if (p.block_sizes) lim = min(lim, p.block_sizes[b * p.bs_stride_b + h * p.bs_stride_h + j]);
  return max(lim, 0);
}

struct BwdSmem {
  static constexpr int kBarBytes = 256;  // 32 mbarriers
  static constexpr int kMisc = 16;
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

// 64 fp32 accumulator columns of one row -> bf16, scaled -> global (128 contiguous bytes)
__device__ __forceinline__ void store_row_half(__nv_bfloat16* dst, const uint32_t* acc, float scale) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    uint4 v;
    v.x = pack_bf16x2(__uint_as_float(acc[ch * 8 + 0]) * scale, __uint_as_float(acc[ch * 8 + 1]) * scale);
    v.y = pack_bf16x2(__uint_as_float(acc[ch * 8 + 2]) * scale, __uint_as_float(acc[ch * 8 + 3]) * scale);
    v.z = pack_bf16x2(__uint_as_float(acc[ch * 8 + 4]) * scale, __uint_as_float(acc[ch * 8 + 5]) * scale);
    v.w = pack_bf16x2(__uint_as_float(acc[ch * 8 + 6]) * scale, __uint_as_float(acc[ch * 8 + 7]) * scale);
    reinterpret_cast<uint4*>(dst)[ch] = v;
  }
}

constexpr uint32_t kIdescKK = umma_idesc(1, 1, 0, 0, 128, 128);   // A K-major, B K-major
// A K-major (smem or tmem), B MN-major with n output columns: the gradients of a 64-wide head take 64-column MMAs
__device__ __forceinline__ uint32_t idesc_kmn(int n) { return umma_idesc(1, 1, 0, 1, 128, (uint32_t)n); }

// The helpers below take ready-made descriptors (built once per kernel); a byte offset b inside a tile is
// an addition of b >> 4 to the descriptor's low word.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr) { return umma_desc_sw128(saddr, 0, 1024); }
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr) { return umma_desc_sw128(saddr, kSlab, 1024); }
constexpr uint64_t kTileDescStep = kTile >> 4;  // descriptor distance between consecutive ring tiles

// D = A(smem, K-major) * B(smem, K-major)^T over the head dimension: `ksteps` = D / 16 k-steps across two slabs
// (a 64-wide head contracts over the first slab only; the zero-filled second one is never read).
// All helpers are called by the whole (converged) issuing warp; only the lane with led != 0 issues.
__device__ __forceinline__ void mma_ss_kk(uint32_t d, uint64_t a_desc, uint64_t b_desc, bool acc, uint32_t led,
                                          int ksteps) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint64_t off = (uint64_t)((k >> 2) * (kSlab >> 4) + (k & 3) * 2);
    umma_f16_ss_led(d, a_desc + off, b_desc + off, kIdescKK, (acc || k > 0) ? 1u : 0u, (k < ksteps) ? led : 0u);
  }
}
// D (+)= A(tmem bf16, two 32-column halves at a_lo / a_hi) * B(smem MN-major)
__device__ __forceinline__ void mma_ts_kmn(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint64_t b_desc_mn, bool acc,
                                           uint32_t led, uint32_t idesc) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t a = (k < 4) ? (a_lo + (uint32_t)k * 8u) : (a_hi + (uint32_t)(k - 4) * 8u);
    umma_f16_ts_led(d, a, b_desc_mn + (uint64_t)(k * 128), idesc, (acc || k > 0) ? 1u : 0u, led);
  }
}

// ------------------------------------------------------------------------------------------------
// 2. dQ kernel
// ------------------------------------------------------------------------------------------------
// smem: Q | dO | ring of 5 tiles (K_0, V_0, K_1, V_1, ...) | barriers | misc.  Q and dO stay in their buffers for
// the whole tile (the S and dP MMAs read them from shared memory) and are released after the tile's last S / dP
// MMA, about one iteration before the tile ends, so the next tile's Q and dO arrive under the last iteration.
// Tensor memory: S @0, dP / dS buffer 0 @128, buffer 1 @256 (dS overwrites the head of each group's half), dQ @384.
// Nothing an MMA produces for iteration j+1 depends on what the compute threads produce in iteration j:
// S is single-buffered but S_{j+1} is issued as soon as every compute thread has loaded S_j into registers, and
// dP_{j+1} goes to the buffer that dQ_{j-1} has finished reading, so both run under the arithmetic of iteration j
// and the compute threads wait for neither in steady state.
constexpr int kDqStages = 5;  // K / V ring; Q and dO have a buffer each in front of it
constexpr int kDqSmem = (2 + kDqStages) * kTile + BwdSmem::kBarBytes + BwdSmem::kMisc;

// BLK = 64: the query tile has 64 rows (top half of the 128-row MMAs, lanes 64-127 idle) and one KV iteration
// gathers two 64-token blocks into a 128-token tile (an odd count re-loads the last block as a masked phantom);
// compute group g then owns exactly block g of the pair.
template <int BLK>
__global__ void __launch_bounds__(kDqThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
              const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const BwdParams p) {
  constexpr int NS = kDqStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sQ = smem_raw;
  uint8_t* sdO = sQ + kTile;
  uint8_t* sRing = sdO + kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRing + NS * kTile);
  uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(bars + 32);
  volatile int& s_abort = *reinterpret_cast<volatile int*>(bars + 33);
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0 && atomicCAS(p.status, 0, (int)kStatusBadIndex) == 0) p.status[2] = 998;
    return;
  }
  const uint32_t bar_base = smem_u32(bars);
  auto BAR = [&](int i) { return bar_base + (uint32_t)i * 8u; };
  // ring_full[NS], ring_empty[NS], q_full, q_empty, do_full, do_empty, s_full, s_free, dp_full[2], ds_full[2],
  // ds_used[2], dq_final, dq_free
  constexpr int kRFull = 0, kREmpty = NS, kQFull = 2 * NS, kQEmpty = kQFull + 1, kDoFull = kQEmpty + 1,
                kDoEmpty = kDoFull + 1, kSFull = kDoEmpty + 1, kSFree = kSFull + 1, kDpFull = kSFree + 1,
                kDsFull = kDpFull + 2, kDsUsed = kDsFull + 2, kDqFinal = kDsUsed + 2, kDqFree = kDqFinal + 1,
                kNumBars = kDqFree + 1;
  static_assert(kNumBars <= 32, "barrier slots");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wctx{&s_abort, p.status};
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < NS; ++i) {
      mbar_init(BAR(kRFull + i), 1);
      mbar_init(BAR(kREmpty + i), 3);  // released once by each issuing warp
    }
    mbar_init(BAR(kQFull), 1);
    mbar_init(BAR(kQEmpty), 1);
    mbar_init(BAR(kDoFull), 1);
    mbar_init(BAR(kDoEmpty), 1);
    mbar_init(BAR(kSFull), 1);
    mbar_init(BAR(kSFree), 256);   // every compute thread has loaded its part of S_j: S_{j+1} may overwrite it
    for (int i = 0; i < 2; ++i) {  // the two dP / dS buffers, by iteration parity
      mbar_init(BAR(kDpFull + i), 1);
      mbar_init(BAR(kDsFull + i), 256);
      mbar_init(BAR(kDsUsed + i), 1);  // the dQ MMAs have read dS from the buffer: it may take the dP after next
    }
    mbar_init(BAR(kDqFinal), 1);
    mbar_init(BAR(kDqFree), 256);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == kBwdMmaWarp) {
    tmem_alloc(smem_u32(&s_tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const uint32_t tS = tmem, tdP = tmem + 128u, tdQ = tmem + 384u;  // dP / dS buffer i at tdP + 128 i
  const int num_work = p.B * p.H * p.Nq;

  constexpr int kPerIt = 128 / BLK;               // KV blocks per 128-token iteration
  constexpr uint32_t kQBytes = 2u * BLK * 128u;   // bytes of a Q (or dO) tile: two slabs of BLK rows
  auto row_count = [&](int w) {
    int c = p.q2k_nums ? p.q2k_nums[w] : p.fixed_count;
    return max(0, min(c, p.cap));
  };
  auto iterations = [&](int count) { return (count + kPerIt - 1) / kPerIt; };
  // ring positions of a tile with n iterations: K_j at +2j and V_j at +2j+1

  if (warp == kDqLoadWarp) {
    uint32_t r_cnt = 0, tile_cnt = 0;
    bool ok = true;
    for (int band = 0; band * (int)gridDim.x < num_work && ok; ++band) {
      const int w = bwd_work_at(p.order_q, band, num_work, p.status);
      if (w < 0) continue;
      const int cnt = row_count(w);
      const int n = iterations(cnt);
      if (n == 0) continue;
      const int m = w % p.Nq;
      const int h = (w / p.Nq) % p.H;
      const int b = w / (p.Nq * p.H);
      const int32_t* row = p.q2k_index + (long long)w * p.cap;
      for (int which = 0; which < 2 && ok; ++which) {  // Q, dO
        const int full = which ? kDoFull : kQFull, empty = which ? kDoEmpty : kQEmpty;
        ok = mbar_wait(BAR(empty), (tile_cnt & 1) ^ 1, wctx, 400);
        if (!ok) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(BAR(full), kQBytes);
          const CUtensorMap* tm = which ? &tm_do : &tm_q;
          for (int sl = 0; sl < 2; ++sl)
            tma_load_4d(smem_u32((which ? sdO : sQ) + sl * kSlab), tm, BAR(full), sl * 64, m * BLK, h, b);
        }
      }
      ++tile_cnt;
      for (int j = 0; j < n && ok; ++j) {
        const int blk0 = row[kPerIt * j];
        const int blk1 = (BLK == 64 && 2 * j + 1 < cnt) ? row[2 * j + 1] : blk0;
        for (int which = 0; which < 2 && ok; ++which) {
          const uint32_t stage = r_cnt % NS, ph = (r_cnt / NS) & 1;
          ok = mbar_wait(BAR(kREmpty + stage), ph ^ 1, wctx, 401);
          if (!ok) break;
          if (lane == 0) {
            mbar_arrive_expect_tx(BAR(kRFull + stage), kTile);
            const CUtensorMap* tm = which ? &tm_v : &tm_k;
            for (int sl = 0; sl < 2; ++sl) {
              const uint32_t dst = smem_u32(sRing + stage * kTile + sl * kSlab);
              tma_load_4d(dst, tm, BAR(kRFull + stage), sl * 64, blk0 * BLK, h, b);
              if (BLK == 64) tma_load_4d(dst + 64 * 128, tm, BAR(kRFull + stage), sl * 64, blk1 * 64, h, b);
            }
          }
          ++r_cnt;
        }
      }
    }
  } else if (warp >= kBwdMmaWarp && warp < kBwdMmaWarp + 3) {
    // Three issuing warps, one per dependency chain (a thread that issues MMAs is stalled at their execution rate,
    // so one thread issuing S and dP in turn delivers S late):
    //   issuer 0: S_j = Q K_j^T; S_{j+1} once every compute thread holds S_j in registers.
    //   issuer 1: dQ += dS_j K_j.
    //   issuer 2: dP_j = dO V_j^T; dP_{j+1} (buffer (j+1) & 1) once dQ_{j-1} has read dS_{j-1} from that buffer.
    // Neither S nor dP waits for anything the compute threads produce in the running iteration.
    // All three visit every ring position in increasing order and release every stage once (a commit after the last MMA
    // that reads the tile, a plain arrival for a tile the issuer does not read).
    const int who = warp - kBwdMmaWarp;
    uint32_t r_cnt = 0, free_cnt = 0, s_issued = 0, dp_issued = 0, ds_seen = 0, tile_cnt = 0;
    bool ok = true;
    bool first_tile = true;
    const uint32_t led = lane == 0;  // the whole warp runs the issue code, this lane issues
    const uint64_t ring_k = desc_k_major(smem_u32(sRing)), ring_mn = desc_mn_major(smem_u32(sRing));
    const int ksteps = p.D / 16;              // contraction steps of S and dP
    const uint32_t idesc_n = idesc_kmn(p.D);  // dQ has D columns
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < num_work && ok; ++band) {
      const int w = bwd_work_at(p.order_q, band, num_work, p.status);
      if (w < 0) continue;
      const int n = iterations(row_count(w));
      if (n == 0) continue;
      const uint32_t base = r_cnt;  // K_j at base + 2j, V_j at base + 2j + 1
      auto stage_of = [&](uint32_t pos) { return pos % NS; };
      auto wait_full = [&](uint32_t pos) {
        PT_MARK(0)
        const bool r = mbar_wait(BAR(kRFull + stage_of(pos)), (pos / NS) & 1, wctx, 411);
        PT_MARK(2)
        return r;
      };
      auto pass = [&](uint32_t pos) {  // a tile this issuer does not read
        if (!wait_full(pos)) return false;
        if (led) mbar_arrive(BAR(kREmpty + stage_of(pos)));
        __syncwarp();
        return true;
      };
      if (who == 0) {
        PT_MARK(0)
        ok = mbar_wait(BAR(kQFull), tile_cnt & 1, wctx, 410);
        PT_MARK(1)
        const uint64_t q_desc = desc_k_major(smem_u32(sQ));
        for (int j = 0; j < n && ok; ++j) {
          ok = wait_full(base + 2 * j);  // K_j
          if (!ok) break;
          if (s_issued > 0) {  // the previous S has been loaded into registers by every compute thread
            PT_MARK(0)
            ok = mbar_wait(BAR(kSFree), (s_issued - 1) & 1, wctx, 414);
            if (!ok) break;
            PT_MARK(5)
          }
          ++s_issued;
          tc_fence_after();
          {
            const uint32_t sk = stage_of(base + 2 * j);
            mma_ss_kk(tS, q_desc, ring_k + sk * kTileDescStep, false, led, ksteps);
            umma_commit_led(BAR(kSFull), led);
            umma_commit_led(BAR(kREmpty + sk), led);
            if (j == n - 1) umma_commit_led(BAR(kQEmpty), led);  // the tile's last S: Q may be replaced
          }
          __syncwarp();
          ok = pass(base + 2 * j + 1);  // V_j
        }
        if (!ok) break;
      } else if (who == 2) {
        PT_MARK(0)
        ok = mbar_wait(BAR(kDoFull), tile_cnt & 1, wctx, 416);
        PT_MARK(1)
        const uint64_t do_desc = desc_k_major(smem_u32(sdO));
        for (int j = 0; j < n && ok; ++j) {
          ok = pass(base + 2 * j);  // K_j
          if (ok) ok = wait_full(base + 2 * j + 1);  // V_j
          if (!ok) break;
          const uint32_t buf = dp_issued & 1;
          if (dp_issued >= 2) {  // dS of two iterations back has been read from this buffer
            PT_MARK(0)
            ok = mbar_wait(BAR(kDsUsed + buf), ((dp_issued >> 1) - 1) & 1, wctx, 415);
            if (!ok) break;
            PT_MARK(3)
          }
          ++dp_issued;
          tc_fence_after();
          {
            const uint32_t sv = stage_of(base + 2 * j + 1);
            mma_ss_kk(tdP + buf * 128u, do_desc, ring_k + sv * kTileDescStep, false, led, ksteps);
            umma_commit_led(BAR(kDpFull + buf), led);
            umma_commit_led(BAR(kREmpty + sv), led);
            if (j == n - 1) umma_commit_led(BAR(kDoEmpty), led);  // the tile's last dP: dO may be replaced
          }
          __syncwarp();
        }
        if (!ok) break;
      } else {
        for (int j = 0; j < n && ok; ++j) {
          ok = wait_full(base + 2 * j);  // K_j
          if (ok) ok = pass(base + 2 * j + 1);  // V_j
          if (!ok) break;
          const uint32_t buf = ds_seen & 1;
          PT_MARK(0)
          ok = mbar_wait(BAR(kDsFull + buf), (ds_seen >> 1) & 1, wctx, 412);  // dS_j in tensor memory
          if (!ok) break;
          PT_MARK(3)
          ++ds_seen;
          if (j == 0 && !first_tile) {  // the previous tile's epilogue has drained dQ
            PT_MARK(0)
            ok = mbar_wait(BAR(kDqFree), free_cnt & 1, wctx, 413);
            if (!ok) break;
            PT_MARK(4)
            ++free_cnt;
          }
          tc_fence_after();
          {
            const uint32_t sk = stage_of(base + 2 * j);
            // dQ += dS_j (bf16 in tensor memory, at the head of each group's half of the buffer) * K_j
            // (MN-major view of the K tile)
            const uint32_t t = tdP + buf * 128u;
            mma_ts_kmn(tdQ, t, t + 64u, ring_mn + sk * kTileDescStep, j > 0, led, idesc_n);
            umma_commit_led(BAR(kDsUsed + buf), led);
            umma_commit_led(BAR(kREmpty + sk), led);
          }
          __syncwarp();
        }
        if (!ok) break;
        umma_commit_led(BAR(kDqFinal), led);
        __syncwarp();
      }
      r_cnt += 2 * n;
      ++tile_cnt;
      first_tile = false;
    }
    PT_MARK(0)
    if (who == 0) { PTB_FLUSH(16) } else if (who == 1) { PTB_FLUSH(24) } else { PTB_FLUSH(32) }
  } else if (warp < 8) {
    const int grp = warp >> 2;
    const int row = threadIdx.x & 127;
    const bool row_active = (BLK == 128) || (row < 64);  // warp-uniform
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t s_cnt = 0, dp_cnt = 0, fin_cnt = 0;
    bool ok = true;
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < num_work && ok; ++band) {
      const int w = bwd_work_at(p.order_q, band, num_work, p.status);
      if (w < 0) continue;
      const int cnt = row_count(w);
      const int n = iterations(cnt);
      const int m = w % p.Nq;
      const int h = (w / p.Nq) % p.H;
      const int b = w / (p.Nq * p.H);
      const int seq = m * BLK + row;
      __nv_bfloat16* dq_row = p.dq + b * p.dq_stride[0] + h * p.dq_stride[1] + (long long)seq * p.dq_stride[2] + grp * 64;
      if (n == 0) {
        if (row_active && seq < p.Sq && grp * 64 < p.D) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) reinterpret_cast<uint4*>(dq_row)[ch] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const long long srow = ((long long)b * p.H + h) * ((long long)p.Nq * BLK) + seq;
      const float nlse = row_active ? p.lse_log2[srow] : -INFINITY;  // negated statistics, see the preprocess
      const float ndlt = row_active ? p.delta[srow] : 0.f;
      const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), nl2 = pack2(nlse, nlse), nd2 = pack2(ndlt, ndlt);
      const int32_t* idx_row = p.q2k_index + (long long)w * p.cap;
      // valid kv tokens among this group's 64 columns of the 128-token tile of iteration j; fetched one iteration
      // ahead so that the index load never sits in front of the arithmetic
      auto valid_len = [&](int j) -> int {
        if (BLK == 128) return bwd_block_len<128>(p, b, h, idx_row[j]) - grp * 64;
        return (2 * j + grp < cnt) ? bwd_block_len<64>(p, b, h, idx_row[2 * j + grp]) : 0;
      };
      int len_next = valid_len(0);
      for (int j = 0; j < n && ok; ++j) {
        const int len = len_next;
        // ---- phase 1: P = exp2(S*scale - lse)
        PT_MARK(0)
        ok = mbar_wait(BAR(kSFull), s_cnt & 1, wctx, 420);
        if (!ok) break;
        PT_MARK(1)
        ++s_cnt;
        tc_fence_after();
        const uint32_t buf = dp_cnt & 1;  // dP / dS buffer of this iteration
        if (!row_active) {  // idle half of a 64-row tile: barrier protocol only
          mbar_arrive(BAR(kSFree));
          ok = mbar_wait(BAR(kDpFull + buf), (dp_cnt >> 1) & 1, wctx, 421);
          if (!ok) break;
          ++dp_cnt;
          tc_fence_before();
          mbar_arrive(BAR(kDsFull + buf));
          continue;
        }
        float pr[64];
        {
          uint32_t* u = reinterpret_cast<uint32_t*>(pr);
          tmem_ld32(tS + lane_base + grp * 64, u);
          tmem_ld32(tS + lane_base + grp * 64 + 32, u + 32);
          tmem_wait_ld();
        }
        tc_fence_before();
        mbar_arrive(BAR(kSFree));  // S_j is in registers: the next S may be computed
        if (j + 1 < n) len_next = valid_len(j + 1);
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float x0, x1;
          unpack2(ffma2(pack2(pr[c], pr[c + 1]), sc2, nl2), x0, x1);
          pr[c] = ex2_approx(x0);
          pr[c + 1] = ex2_approx(x1);
        }
        if (len < 64) {
#pragma unroll
          for (int c = 0; c < 64; ++c) pr[c] = (c < len) ? pr[c] : 0.f;
        }
        // ---- phase 2: dS = P o (dP - delta) -> bf16 -> tensor memory (head of this group's half of the buffer)
        PT_MARK(2)
        ok = mbar_wait(BAR(kDpFull + buf), (dp_cnt >> 1) & 1, wctx, 421);
        if (!ok) break;
        PT_MARK(3)
        ++dp_cnt;
        tc_fence_after();
        const uint32_t tbuf = tdP + buf * 128u + lane_base + grp * 64;
        uint32_t dp[64];
        tmem_ld32(tbuf, dp);
        tmem_ld32(tbuf + 32, dp + 32);
        tmem_wait_ld();
        {
          uint32_t pk[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float d0, d1;
            unpack2(fmul2(pack2(pr[2 * e], pr[2 * e + 1]),
                          fadd2(pack2(__uint_as_float(dp[2 * e]), __uint_as_float(dp[2 * e + 1])), nd2)), d0, d1);
            pk[e] = pack_bf16x2(d0, d1);
          }
          tmem_st32(tbuf, pk);
          tmem_wait_st();
        }
        tc_fence_before();
        mbar_arrive(BAR(kDsFull + buf));
        PT_MARK(4)
      }
      if (!ok) break;
      // ---- epilogue: dQ * softmax_scale -> bf16 -> global
      ok = mbar_wait(BAR(kDqFinal), fin_cnt & 1, wctx, 422);
      if (!ok) break;
      ++fin_cnt;
      tc_fence_after();
      uint32_t acc[64];
      if (row_active) {
        tmem_ld32(tdQ + lane_base + grp * 64, acc);
        tmem_ld32(tdQ + lane_base + grp * 64 + 32, acc + 32);
        tmem_wait_ld();
      }
      tc_fence_before();
      mbar_arrive(BAR(kDqFree));
      if (row_active && seq < p.Sq && grp * 64 < p.D) store_row_half(dq_row, acc, p.softmax_scale);
      PT_MARK(5)
    }
    if ((warp & 3) == 0) { PTB_FLUSH(grp * 8) }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kBwdMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// 3. dK/dV kernel
// ------------------------------------------------------------------------------------------------
// smem: K | V | ring of 5 tiles (Q_i, dO_i alternating) | row statistics [2][2][128] f32 | barriers | misc
// Tensor memory: S @0 takes S^T_i; the next one is issued as soon as every compute thread holds S^T_i in registers,
// i.e. one tile ahead of the compute threads.  G @128 takes dP^T_i and, once a compute thread holds its 64 columns
// of it in registers, that thread's P^T_i (bf16, first 32 of its columns) and dS^T_i (last 32): the tensor-memory
// operands of dV @256 += P^T dO and dK @384 += dS^T Q.  dP^T_{i+1} follows dK_i in the issuing thread's program
// order and waits for the commit behind dV_i (issued by the other warp).
constexpr int kDkvStages = 5;
constexpr int kStatSlots = 2;
constexpr int kDkvSmem = 2 * kTile + kDkvStages * kTile + kStatSlots * 1024 + BwdSmem::kBarBytes + BwdSmem::kMisc;

// BLK = 64: the KV block has 64 tokens (top half of the 128-row MMAs, lanes 64-127 idle) and one iteration
// covers two CSR entries: their 64-row Q / dO tiles form one 128-row ring tile, so compute group g owns
// entry g of the pair (an odd total re-loads the last entry as a masked phantom).
template <int BLK>
__global__ void __launch_bounds__(kDkvThreads, 1)
bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const BwdParams p) {
  constexpr int NS = kDkvStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sK = smem_raw;
  uint8_t* sV = sK + kTile;
  uint8_t* sRing = sV + kTile;
  float* sStats = reinterpret_cast<float*>(sRing + NS * kTile);  // [slot][0: lse_log2, 1: delta][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStats) + kStatSlots * 1024);
  uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(bars + 32);
  volatile int& s_abort = *reinterpret_cast<volatile int*>(bars + 33);
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0 && atomicCAS(p.status, 0, (int)kStatusBadIndex) == 0) p.status[2] = 997;
    return;
  }
  const uint32_t bar_base = smem_u32(bars);
  auto BAR = [&](int i) { return bar_base + (uint32_t)i * 8u; };
  // kv_full, kv_empty, ring_full[NS], ring_empty[NS], s_full, s_free, dp_full, p_full, ds_full, fin, free
  constexpr int kKvFull = 0, kKvEmpty = 1, kRFull = 2, kREmpty = 2 + NS, kSFull = 2 + 2 * NS, kSFree = kSFull + 1,
                kDpFull = kSFree + 1, kPFull = kDpFull + 1, kDsFull = kPFull + 1, kGFree = kDsFull + 1,
                kFinal = kGFree + 1, kFree = kFinal + 1, kNumBars = kFree + 1;
  static_assert(kNumBars <= 32, "barrier slots");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wctx{&s_abort, p.status};
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(BAR(kKvFull), 1);
    mbar_init(BAR(kKvEmpty), 2);  // one commit per issuing warp
    for (int i = 0; i < NS; ++i) {
      mbar_init(BAR(kRFull + i), 1);
      mbar_init(BAR(kREmpty + i), 2);  // released by both issuing warps
    }
    mbar_init(BAR(kSFull), 1);
    mbar_init(BAR(kDpFull), 1);
    mbar_init(BAR(kSFree), 256);   // every compute thread holds its part of S^T_i in registers
    mbar_init(BAR(kPFull), 256);   // ... has stored its part of P^T_i
    mbar_init(BAR(kDsFull), 256);  // ... and of dS^T_i
    mbar_init(BAR(kGFree), 1);     // dV_i has read P^T_i: region G may take dP^T_{i+1} (once dK_i is issued too)
    mbar_init(BAR(kFinal), 2);
    mbar_init(BAR(kFree), 256);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == kBwdMmaWarp) {
    tmem_alloc(smem_u32(&s_tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const uint32_t tS = tmem, tG = tmem + 128u, tdV = tmem + 256u, tdK = tmem + 384u;
  const int num_work = p.B * p.H * p.Nkv;

  constexpr int kPerIt = 128 / BLK;              // CSR entries per 128-row iteration
  constexpr uint32_t kKvBytes = 2u * BLK * 128u;  // bytes of the K (or V) block: two slabs of BLK rows
  auto iterations = [&](int entries) { return (entries + kPerIt - 1) / kPerIt; };
  // number of query tiles attending kv block nb of (b,h): the CSR rows of all query groups
  auto total_rows = [&](int bh, int nb) {
    int t = 0;
    for (int g = 0; g < p.G; ++g) {
      const int32_t* off = p.csr_offsets + ((long long)bh * p.G + g) * (p.Nkv + 1);
      t += off[nb + 1] - off[nb];
    }
    return t;
  };

  if (warp == kDkvLoadWarp) {
    uint32_t r_cnt = 0, kv_cnt = 0, tile_cnt = 0;
    bool ok = true;
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < num_work && ok; ++band) {
      const int w = bwd_work_at(p.order_kv, band, num_work, p.status);
      if (w < 0) continue;
      const int nb = w % p.Nkv;
      const int bh = w / p.Nkv;
      const int h = bh % p.H, b = bh / p.H;
      if (total_rows(bh, nb) == 0) continue;
      PT_MARK(0)
      ok = mbar_wait(BAR(kKvEmpty), (kv_cnt & 1) ^ 1, wctx, 500);
      PT_MARK(1)
      if (!ok) break;
      ++kv_cnt;
      if (lane == 0) {
        mbar_arrive_expect_tx(BAR(kKvFull), 2 * kKvBytes);
        for (int sl = 0; sl < 2; ++sl) {
          tma_load_4d(smem_u32(sK + sl * kSlab), &tm_k, BAR(kKvFull), sl * 64, nb * BLK, h, b);
          tma_load_4d(smem_u32(sV + sl * kSlab), &tm_v, BAR(kKvFull), sl * 64, nb * BLK, h, b);
        }
      }
      // one ring tile pair (Q, dO) for the query blocks qa (rows 0..BLK) and, with 64-token blocks, qb
      auto load_pair = [&](int qa, int qb) -> bool {
        for (int which = 0; which < 2; ++which) {
          const uint32_t stage = r_cnt % NS, ph = (r_cnt / NS) & 1;
          PT_MARK(0)
          if (!mbar_wait(BAR(kREmpty + stage), ph ^ 1, wctx, 501)) return false;
          if (which) { PT_MARK(3) } else { PT_MARK(2) }
          if (lane == 0) {
            const CUtensorMap* tm = which ? &tm_do : &tm_q;
            mbar_arrive_expect_tx(BAR(kRFull + stage), kTile + (which ? 1024 : 0));
            for (int sl = 0; sl < 2; ++sl) {
              const uint32_t dst = smem_u32(sRing + stage * kTile + sl * kSlab);
              tma_load_4d(dst, tm, BAR(kRFull + stage), sl * 64, qa * BLK, h, b);
              if (BLK == 64) tma_load_4d(dst + 64 * 128, tm, BAR(kRFull + stage), sl * 64, qb * 64, h, b);
            }
            if (which) {
              // row statistics of the query rows travel with their dO tile: that stage is re-used only after
              // dK of the tile two back, when the statistics slot of that tile is long free (two slots)
              float* st = sStats + (tile_cnt % kStatSlots) * 256;
              const long long plane = (long long)bh * ((long long)p.Nq * BLK);
              if (BLK == 128) {
                bulk_load_1d(smem_u32(st), p.lse_log2 + plane + (long long)qa * 128, 512, BAR(kRFull + stage));
                bulk_load_1d(smem_u32(st + 128), p.delta + plane + (long long)qa * 128, 512, BAR(kRFull + stage));
              } else {
                bulk_load_1d(smem_u32(st), p.lse_log2 + plane + (long long)qa * 64, 256, BAR(kRFull + stage));
                bulk_load_1d(smem_u32(st + 64), p.lse_log2 + plane + (long long)qb * 64, 256, BAR(kRFull + stage));
                bulk_load_1d(smem_u32(st + 128), p.delta + plane + (long long)qa * 64, 256, BAR(kRFull + stage));
                bulk_load_1d(smem_u32(st + 192), p.delta + plane + (long long)qb * 64, 256, BAR(kRFull + stage));
              }
            }
          }
          ++r_cnt;
        }
        ++tile_cnt;
        return true;
      };
      int pending = -1;  // first entry of an unfinished pair (64-token blocks)
      for (int g = 0; g < p.G && ok; ++g) {
        const int32_t* off = p.csr_offsets + ((long long)bh * p.G + g) * (p.Nkv + 1);
        const int beg = off[nb], end = off[nb + 1];
        for (int e = beg; e < end && ok; ++e) {
          const int qi = p.csr_indices[(long long)bh * p.idx_cap + e];
          if (BLK == 128) {
            ok = load_pair(qi, qi);
          } else if (pending < 0) {
            pending = qi;
          } else {
            ok = load_pair(pending, qi);
            pending = -1;
          }
        }
      }
      if (ok && pending >= 0) ok = load_pair(pending, pending);  // odd total: masked phantom second half
    }
    PT_MARK(0)
    PTB_FLUSH(64 + 32)
  } else if (warp == kBwdMmaWarp || warp == kBwdMmaWarp + 1) {
    // Two issuing warps:
    //   issuer 0: S^T_i = K Q_i^T into region S as soon as every compute thread holds S^T_{i-1} in registers, i.e.
    //             one tile ahead of the compute threads, whose exponentials therefore never wait for it; and
    //             dV += P^T_i dO_i as soon as P^T_i is stored (nothing waits for dV, so it stays off the other chain);
    //   issuer 1: the chain through region G.  dP^T_i = V dO_i^T, then (the compute threads having replaced it by
    //             P^T_i and dS^T_i) dK += dS^T_i Q_i and, behind it in program order and once dV_i has completed
    //             (g_free), dP^T_{i+1}.
    // Each issuer releases every ring stage once, by a commit after its last MMA on the tile.
    const int who = warp - kBwdMmaWarp;
    const uint32_t led = lane == 0;  // the whole warp runs the issue code, this lane issues
    uint32_t r_cnt = 0, kv_cnt = 0, in_cnt = 0, ds_cnt = 0, free_cnt = 0;
    bool ok = true, first_item = true;
    const uint64_t k_desc = desc_k_major(smem_u32(sK)), v_desc = desc_k_major(smem_u32(sV));
    const uint64_t ring_k = desc_k_major(smem_u32(sRing)), ring_mn = desc_mn_major(smem_u32(sRing));
    const int ksteps = p.D / 16;              // contraction steps of S^T and dP^T
    const uint32_t idesc_n = idesc_kmn(p.D);  // dK and dV have D columns
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < num_work && ok; ++band) {
      const int w = bwd_work_at(p.order_kv, band, num_work, p.status);
      if (w < 0) continue;
      const int nb = w % p.Nkv;
      const int bh = w / p.Nkv;
      const int T = iterations(total_rows(bh, nb));
      if (T == 0) continue;
      ok = mbar_wait(BAR(kKvFull), kv_cnt & 1, wctx, 510);
      if (!ok) break;
      ++kv_cnt;
      const uint32_t base = r_cnt;  // Q_i at base+2i, dO_i at base+2i+1
      auto stage_of = [&](uint32_t pos) { return pos % NS; };
      auto wait_full = [&](uint32_t pos) {
        PT_MARK(0)
        const bool r = mbar_wait(BAR(kRFull + stage_of(pos)), (pos / NS) & 1, wctx, 511);
        if (pos & 1u) { PT_MARK(2) } else { PT_MARK(1) }  // (base is even: odd positions are dO tiles)
        return r;
      };
      auto wait_free = [&]() -> bool {  // the previous item's epilogue has drained the accumulators
        if (first_item) return true;
        const bool r = mbar_wait(BAR(kFree), free_cnt & 1, wctx, 515);
        ++free_cnt;
        return r;
      };
      if (who == 0) {
        // S^T_{i+1} as soon as S^T_i is in registers, dV_i as soon as P^T_i is stored
        auto issue_st = [&](int i) -> bool {
          if (!wait_full(base + 2 * i)) return false;  // Q_i
          if (in_cnt > 0) {  // S^T of the tile before (of this or the previous item) is in registers
            PT_MARK(0)
            const bool r = mbar_wait(BAR(kSFree), (in_cnt - 1) & 1, wctx, 512);
            PT_MARK(3)
            if (!r) return false;
          }
          ++in_cnt;
          tc_fence_after();
          const uint32_t sq = stage_of(base + 2 * i);
          mma_ss_kk(tS, k_desc, ring_k + sq * kTileDescStep, false, led, ksteps);  // S^T_i
          umma_commit_led(BAR(kSFull), led);
          umma_commit_led(BAR(kREmpty + sq), led);
          __syncwarp();
          PT_MARK(5)
          return true;
        };
        ok = issue_st(0);
        for (int i = 0; i < T && ok; ++i) {
          if (i + 1 < T) ok = issue_st(i + 1);
          if (ok) ok = wait_full(base + 2 * i + 1);  // dO_i
          if (!ok) break;
          PT_MARK(0)
          ok = mbar_wait(BAR(kPFull), ds_cnt & 1, wctx, 513);  // P^T_i in region G
          ++ds_cnt;
          PT_MARK(4)
          if (ok && i == 0) ok = wait_free();
          if (!ok) break;
          tc_fence_after();
          {
            const uint32_t sd = stage_of(base + 2 * i + 1);
            mma_ts_kmn(tdV, tG, tG + 64u, ring_mn + sd * kTileDescStep, i > 0, led, idesc_n);  // dV += P^T_i dO_i
            umma_commit_led(BAR(kREmpty + sd), led);
            umma_commit_led(BAR(kGFree), led);
          }
          __syncwarp();
          PT_MARK(6)
        }
      } else {
        auto issue_dp = [&](int i) -> bool {
          if (!wait_full(base + 2 * i)) return false;      // Q_i: read by dK_i later
          if (!wait_full(base + 2 * i + 1)) return false;  // dO_i
          const uint32_t sd = stage_of(base + 2 * i + 1);
          mma_ss_kk(tG, v_desc, ring_k + sd * kTileDescStep, false, led, ksteps);  // dP^T_i
          umma_commit_led(BAR(kDpFull), led);
          umma_commit_led(BAR(kREmpty + sd), led);
          __syncwarp();
          PT_MARK(7)
          return true;
        };
        ok = issue_dp(0);
        for (int i = 0; i < T && ok; ++i) {
          PT_MARK(0)
          ok = mbar_wait(BAR(kDsFull), ds_cnt & 1, wctx, 514);  // dS^T_i in region G
          ++ds_cnt;
          PT_MARK(4)
          if (ok && i == 0) ok = wait_free();
          if (!ok) break;
          tc_fence_after();
          {
            const uint32_t sq = stage_of(base + 2 * i);
            mma_ts_kmn(tdK, tG + 32u, tG + 96u, ring_mn + sq * kTileDescStep, i > 0, led, idesc_n);  // dK += dS^T_i Q_i
            umma_commit_led(BAR(kREmpty + sq), led);
          }
          __syncwarp();
          PT_MARK(5)
          // dV_i (issued by the other warp when P^T_i was stored) has read region G as well
          ok = mbar_wait(BAR(kGFree), in_cnt & 1, wctx, 516);
          ++in_cnt;
          PT_MARK(3)
          if (ok && i + 1 < T) ok = issue_dp(i + 1);
        }
      }
      if (!ok) break;
      {  // both issuers: their share of the accumulators is final, K / V no longer needed
        umma_commit_led(BAR(kFinal), led);
        umma_commit_led(BAR(kKvEmpty), led);
      }
      __syncwarp();
      r_cnt += 2 * T;
      first_item = false;
    }
    PT_MARK(0)
    if (who == 0) { PTB_FLUSH(64 + 16) } else { PTB_FLUSH(64 + 24) }
  } else if (warp < 8) {
    const int grp = warp >> 2;
    const int row = threadIdx.x & 127;  // kv token inside the block = tensor-memory lane
    const bool row_active = (BLK == 128) || (row < 64);  // warp-uniform
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t s_cnt = 0, dp_cnt = 0, fin_cnt = 0, tile_cnt = 0, r_cnt = 0;
    const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2);
    bool ok = true;
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < num_work && ok; ++band) {
      const int w = bwd_work_at(p.order_kv, band, num_work, p.status);
      if (w < 0) continue;
      const int nb = w % p.Nkv;
      const int bh = w / p.Nkv;
      const int h = bh % p.H, b = bh / p.H;
      const int entries = total_rows(bh, nb);
      const int T = iterations(entries);
      const uint32_t base = r_cnt;
      r_cnt += 2 * T;
      const int kv = nb * BLK + row;
      const bool kv_valid = row_active && kv < p.Sk && grp * 64 < p.D;  // this thread stores a dK / dV row half
      const bool kv_live = row < bwd_block_len<BLK>(p, b, h, nb);       // the token takes part in the softmax
      __nv_bfloat16* dk_row = p.dk + b * p.dk_stride[0] + h * p.dk_stride[1] + (long long)kv * p.dk_stride[2] + grp * 64;
      __nv_bfloat16* dv_row = p.dv + b * p.dv_stride[0] + h * p.dv_stride[1] + (long long)kv * p.dv_stride[2] + grp * 64;
      if (T == 0) {
        if (kv_valid) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            reinterpret_cast<uint4*>(dk_row)[ch] = make_uint4(0, 0, 0, 0);
            reinterpret_cast<uint4*>(dv_row)[ch] = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      for (int i = 0; i < T && ok; ++i) {
        const float4* st_l = reinterpret_cast<const float4*>(sStats + (tile_cnt % kStatSlots) * 256 + grp * 64);
        const float4* st_d = reinterpret_cast<const float4*>(sStats + (tile_cnt % kStatSlots) * 256 + 128 + grp * 64);
        ++tile_cnt;
        // ---- phase 1: P^T = exp2(S^T*scale - lse[q]) -> bf16 -> Y
        PT_MARK(0)
        ok = mbar_wait(BAR(kSFull), s_cnt & 1, wctx, 520);
        if (!ok) break;
        PT_MARK(1)
        ++s_cnt;
        if (!row_active) {
          // idle half of a 64-token block: barrier protocol only, in exactly the order of the working threads
          // (an arrival for the next phase of a 256-thread barrier must not precede the end of the running one)
          mbar_arrive(BAR(kSFree));
          ok = mbar_wait(BAR(kDpFull), dp_cnt & 1, wctx, 521);
          if (!ok) break;
          ++dp_cnt;
          mbar_arrive(BAR(kPFull));
          mbar_arrive(BAR(kDsFull));
          continue;
        }
        {
          // observe the arrival of this tile's row statistics directly (they were copied on the dO
          // stage's barrier); the phase cannot have advanced further: the stage is held until dV
          const uint32_t pos = base + 2 * (uint32_t)i + 1;
          ok = mbar_wait(BAR(kRFull + pos % NS), (pos / NS) & 1, wctx, 523);
          if (!ok) break;
        }
        PT_MARK(7)
        tc_fence_after();
        float pr[64];
        {
          uint32_t* u = reinterpret_cast<uint32_t*>(pr);
          tmem_ld32(tS + lane_base + grp * 64, u);
          tmem_ld32(tS + lane_base + grp * 64 + 32, u + 32);
          tmem_wait_ld();
        }
        // S^T_i is in registers: region S may take S^T_{i+1}
        tc_fence_before();
        mbar_arrive(BAR(kSFree));
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 l = st_l[c4];  // negated
          float x0, x1, x2, x3;
          unpack2(ffma2(pack2(pr[c4 * 4 + 0], pr[c4 * 4 + 1]), sc2, pack2(l.x, l.y)), x0, x1);
          unpack2(ffma2(pack2(pr[c4 * 4 + 2], pr[c4 * 4 + 3]), sc2, pack2(l.z, l.w)), x2, x3);
          pr[c4 * 4 + 0] = ex2_approx(x0);
          pr[c4 * 4 + 1] = ex2_approx(x1);
          pr[c4 * 4 + 2] = ex2_approx(x2);
          pr[c4 * 4 + 3] = ex2_approx(x3);
        }
        // masked KV token, or the phantom second half of an odd pair
        if (!kv_live || (BLK == 64 && grp == 1 && 2 * i + 1 >= entries)) {
#pragma unroll
          for (int c = 0; c < 64; ++c) pr[c] = 0.f;
        }
        PT_MARK(2)
        // ---- phase 2: dS^T = P^T o (dP^T - delta[q]) -> bf16 -> Y
        ok = mbar_wait(BAR(kDpFull), dp_cnt & 1, wctx, 521);
        if (!ok) break;
        PT_MARK(3)
        ++dp_cnt;
        tc_fence_after();
        uint32_t dp[64];
        tmem_ld32(tG + lane_base + grp * 64, dp);
        tmem_ld32(tG + lane_base + grp * 64 + 32, dp + 32);
        tmem_wait_ld();
        // dP^T_i is in registers: this thread's 64 columns of region G now take P^T_i (bf16, first 32 columns) and
        // dS^T_i (last 32), the tensor-memory operands of dV and dK
#pragma unroll
        for (int h = 0; h < 4; ++h) {  // packed eight registers at a time: pr and dp are both live here
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) pk[e] = pack_bf16x2(pr[16 * h + 2 * e], pr[16 * h + 2 * e + 1]);
          tmem_st8(tG + lane_base + grp * 64 + h * 8, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(BAR(kPFull));
        PT_MARK(6)
        {
          uint32_t pk[32];
#pragma unroll
          for (int c4 = 0; c4 < 16; ++c4) {
            const float4 d = st_d[c4];  // negated
            float d0, d1, d2, d3;
            unpack2(fmul2(pack2(pr[c4 * 4 + 0], pr[c4 * 4 + 1]),
                          fadd2(pack2(__uint_as_float(dp[c4 * 4 + 0]), __uint_as_float(dp[c4 * 4 + 1])), pack2(d.x, d.y))),
                    d0, d1);
            unpack2(fmul2(pack2(pr[c4 * 4 + 2], pr[c4 * 4 + 3]),
                          fadd2(pack2(__uint_as_float(dp[c4 * 4 + 2]), __uint_as_float(dp[c4 * 4 + 3])), pack2(d.z, d.w))),
                    d2, d3);
            pk[c4 * 2] = pack_bf16x2(d0, d1);
            pk[c4 * 2 + 1] = pack_bf16x2(d2, d3);
          }
          tmem_st32(tG + lane_base + grp * 64 + 32, pk);
          tmem_wait_st();
        }
        tc_fence_before();
        mbar_arrive(BAR(kDsFull));
        PT_MARK(4)
      }
      if (!ok) break;
      // ---- epilogue
      ok = mbar_wait(BAR(kFinal), fin_cnt & 1, wctx, 522);
      if (!ok) break;
      ++fin_cnt;
      tc_fence_after();
      uint32_t acc[64];
      if (row_active) {
        tmem_ld32(tdV + lane_base + grp * 64, acc);
        tmem_ld32(tdV + lane_base + grp * 64 + 32, acc + 32);
        tmem_wait_ld();
        if (kv_valid) store_row_half(dv_row, acc, 1.0f);
        tmem_ld32(tdK + lane_base + grp * 64, acc);
        tmem_ld32(tdK + lane_base + grp * 64 + 32, acc + 32);
        tmem_wait_ld();
      }
      tc_fence_before();
      mbar_arrive(BAR(kFree));
      if (kv_valid) store_row_half(dk_row, acc, p.softmax_scale);
      PT_MARK(5)
    }
    if ((warp & 3) == 0) { PTB_FLUSH(64 + grp * 8) }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kBwdMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace bsa

using namespace bsa;

#ifdef BSA_PHASE_TIMERS
// development builds only: copies the backward phase counters to the host and clears them
extern "C" int bsa_bwd_phase_timers(unsigned long long* host_out) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host_out, g_bwd_phase, sizeof(unsigned long long) * 128);
  static unsigned long long zeros[128];
  cudaMemcpyToSymbol(g_bwd_phase, zeros, sizeof(zeros));
  return 0;
}
#endif

extern "C" int64_t bsa_bwd_workspace_bytes(int32_t B, int32_t H, int32_t Sq, int32_t Sk, int32_t D) {
  (void)Sk;
  (void)D;
  if (B < 1 || H < 1 || Sq < 1) return 0;
  const int64_t nq = (Sq + 127) / 128;
  return 2 * (int64_t)B * H * nq * 128 * (int64_t)sizeof(float);
}

extern "C" int bsa_bwd(const bsa_bwd_args* a, void* cuda_stream) {
  if (!a) return set_error(BSA_ERR_INVALID, "bsa_bwd: null args");
  if (a->blk != 128 && a->blk != 64) return set_error(BSA_ERR_UNSUPPORTED, "bsa_bwd: block size %d not built (64 or 128)", a->blk);
  if (a->D != 128 && !(a->D == 64 && a->blk == 128))
    return set_error(BSA_ERR_UNSUPPORTED, "bsa_bwd: head dimension %d not built (128, or 64 with 128-token blocks)", a->D);
  if (a->B < 1 || a->H < 1 || a->Sq < 1 || a->Sk < 1) return set_error(BSA_ERR_INVALID, "bsa_bwd: non-positive extent");
  if (!a->dout || !a->q || !a->k || !a->v || !a->out || !a->lse || !a->dq || !a->dk || !a->dv || !a->q2k_index ||
      !a->csr_offsets || !a->csr_indices || !a->workspace || !a->status)
    return set_error(BSA_ERR_INVALID, "bsa_bwd: null pointer");
  if (a->num_q_groups < 1 || a->cap < 0) return set_error(BSA_ERR_INVALID, "bsa_bwd: bad metadata extents");
  const int64_t need = bsa_bwd_workspace_bytes(a->B, a->H, a->Sq, a->Sk, a->D);
  if (a->workspace_bytes < need) return set_error(BSA_ERR_WORKSPACE, "bsa_bwd: workspace of %lld bytes needed", (long long)need);
  for (int i = 0; i < 3; ++i) {
    if ((a->dq_stride[i] | a->dk_stride[i] | a->dv_stride[i] | a->o_stride[i] | a->do_stride[i]) % 8 != 0)
      return set_error(BSA_ERR_INVALID, "bsa_bwd: strides must be multiples of 8 elements");
  }
  if (a->stages < 0 || a->stages > 7) return set_error(BSA_ERR_INVALID, "bsa_bwd: stages must be a mask of bits 0-2");
  // the preprocess pass and the epilogues use 16-byte vector accesses on these tensors
  {
    const void* vec16[5] = {a->out, a->dout, a->dq, a->dk, a->dv};
    const char* names[5] = {"out", "dout", "dq", "dk", "dv"};
    for (int i = 0; i < 5; ++i)
      if ((reinterpret_cast<uintptr_t>(vec16[i]) & 15u) != 0)
        return set_error(BSA_ERR_INVALID, "%s: base address must be 16-byte aligned", names[i]);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  int dev = 0;
  cudaGetDevice(&dev);
  const int num_sms = bsa_num_sms(dev);
  if (num_sms <= 0) return set_error(BSA_ERR_CUDA, "bsa_bwd: cannot query the SM count");

  const int blk = a->blk;
  const int Nq = (a->Sq + blk - 1) / blk, Nkv = (a->Sk + blk - 1) / blk;
  const long long work_q = (long long)a->B * a->H * Nq, work_kv = (long long)a->B * a->H * Nkv;
  if (work_q > 0x7fffffffLL || work_kv > 0x7fffffffLL) return set_error(BSA_ERR_UNSUPPORTED, "bsa_bwd: too many tiles");
  // every argument is validated (tensor maps included) before the first launch
  CUtensorMap tq, tdo, tk, tv;
  {
    uint64_t qd[4] = {(uint64_t)a->D, (uint64_t)a->Sq, (uint64_t)a->H, (uint64_t)a->B};
    uint64_t kd[4] = {(uint64_t)a->D, (uint64_t)a->Sk, (uint64_t)a->H, (uint64_t)a->B};
    uint32_t box[4] = {64, (uint32_t)blk, 1, 1};
    auto strides = [](const int64_t* s, uint64_t* out) {
      out[0] = (uint64_t)s[2] * 2;
      out[1] = (uint64_t)s[1] * 2;
      out[2] = (uint64_t)s[0] * 2;
    };
    uint64_t sb[3];
    int rc;
    strides(a->q_stride, sb);
    if ((rc = make_tensor_map(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->q, qd, sb, box, "q"))) return rc;
    strides(a->do_stride, sb);
    if ((rc = make_tensor_map(&tdo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->dout, qd, sb, box, "dout"))) return rc;
    strides(a->k_stride, sb);
    if ((rc = make_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->k, kd, sb, box, "k"))) return rc;
    strides(a->v_stride, sb);
    if ((rc = make_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, a->v, kd, sb, box, "v"))) return rc;
  }
  auto* dq_kernel = blk == 128 ? bwd_dq_kernel<128> : bwd_dq_kernel<64>;
  auto* dkv_kernel = blk == 128 ? bwd_dkv_kernel<128> : bwd_dkv_kernel<64>;
  cudaError_t e = cudaFuncSetAttribute(dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmem);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDkvSmem);
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_bwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const int stages = a->stages == 0 ? 7 : a->stages;

  const long long rows_pad = (long long)a->B * a->H * Nq * blk;
  float* lse_log2 = reinterpret_cast<float*>(a->workspace);
  float* delta = lse_log2 + rows_pad;
  if (stages & 1) {
    bwd_preprocess_kernel<<<(unsigned)((rows_pad + 8 * kPreRowsPerWarp - 1) / (8 * kPreRowsPerWarp)), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(a->out), reinterpret_cast<const __nv_bfloat16*>(a->dout), a->lse, lse_log2,
        delta, a->o_stride[0], a->o_stride[1], a->o_stride[2], a->do_stride[0], a->do_stride[1], a->do_stride[2], a->H,
        a->Sq, Nq * blk, rows_pad, a->D);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bwd preprocess launch: %s", cudaGetErrorString(e));
  }
  BwdParams p{};
  p.q2k_index = a->q2k_index;
  p.q2k_nums = a->q2k_nums;
  p.csr_offsets = a->csr_offsets;
  p.csr_indices = a->csr_indices;
  p.order_q = a->work_order_q;
  p.order_kv = a->work_order_kv;
  p.block_sizes = a->block_sizes;
  p.bs_stride_b = a->bs_stride_b;
  p.bs_stride_h = a->bs_stride_h;
  p.lse_log2 = lse_log2;
  p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(a->dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(a->dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(a->dv);
  p.status = a->status;
  for (int i = 0; i < 3; ++i) {
    p.dq_stride[i] = a->dq_stride[i];
    p.dk_stride[i] = a->dk_stride[i];
    p.dv_stride[i] = a->dv_stride[i];
  }
  const long long idx_cap = (long long)Nq * a->cap > 1 ? (long long)Nq * a->cap : 1;
  p.idx_cap = idx_cap;
  p.fixed_count = a->block_sparse_num;
  p.cap = a->cap;
  p.B = a->B;
  p.H = a->H;
  p.Sq = a->Sq;
  p.Sk = a->Sk;
  p.Nq = Nq;
  p.Nkv = Nkv;
  p.G = a->num_q_groups;
  p.D = a->D;
  p.softmax_scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * kLog2e;

  const int grid_q = (int)(work_q < num_sms ? work_q : num_sms);
  const int grid_kv = (int)(work_kv < num_sms ? work_kv : num_sms);
  if (stages & 2) {
    dq_kernel<<<grid_q, kDqThreads, kDqSmem, st>>>(tq, tdo, tk, tv, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bwd dQ launch: %s", cudaGetErrorString(e));
  }
  if (stages & 4) {
    dkv_kernel<<<grid_kv, kDkvThreads, kDkvSmem, st>>>(tq, tdo, tk, tv, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bwd dK/dV launch: %s", cudaGetErrorString(e));
  }
  return BSA_OK;
}
