// Block-sparse attention forward for sm_100a: TMA gathers of the K/V blocks named by the q2k index,
// tcgen05 QK^T and PV MMAs accumulating in tensor memory, online softmax with LSE.
//
// Two persistent CTAs per SM, each walking (q tile, split) work items on its own: while one CTA's softmax
// works on a score tile, the tensor pipe runs the other CTA's MMAs, and a tile boundary (epilogue, first loads)
// of one CTA is covered by the steady state of the other.  Warp roles of a CTA (256 threads):
//   warps 0-3   softmax: one thread per query row (= tensor-memory lane), all 128 score columns of the row
//   warp  4     MMA issue (one lane): QK(0), then PV(i), QK(i+1) per KV iteration
//   warp  5     TMA producer (one lane): Q tile and the K/V ring in consumption order K(0), V(0), K(1), ...
//   warps 6-7   idle; they complete the second warpgroup, whose four warps hand their registers to the softmax
//               warps (setmaxnreg is a warpgroup-wide operation)
// Tensor memory: 256 of the SM's 512 columns per CTA, S @0 and O @128 (fp32, 128 lanes x 128 columns each);
// the probabilities P overwrite the head of S (bf16: 64 columns, e4m3: 32 columns) and are the A operand of
// the PV MMA straight from tensor memory.  S(i+1) is issued behind PV(i) and so may overwrite P(i).
// The output rows leave tensor memory through registers straight to global memory (a thread owns a whole row).
//
// A "KV iteration" is one 128-token tile: one 128-block, or two gathered 64-blocks (the second may be a
// masked phantom when the count is odd).  With 64-token blocks the query tile has 64 rows and sits in
// the top half of the 128-row MMA; lanes 64-127 compute on stale shared memory and are never read.
//
// Semantics follow the reference kernels csrc/fwd/sm100_blk128/bsa_fwd_sm100.py (load order :953-982,
// softmax rules csrc/utils/softmax.py:102-192, merge and LSE :1551-1636) and
// csrc/fwd/sm100_blk64/bsa_fwd_sm100.py; the Sage FP8 scale handling follows
// csrc/fwd/sm100_blk128/bsa_fwd_sm100_fp8_fused_pv.py:1510-1663.
#include "bsa_b200.h"
#include "bsa_common.cuh"
#include "bsa_host.h"

#include <type_traits>

#ifdef BSA_PHASE_TIMERS
// Development builds only (build.py --phase-timers): per-role clock counters, read by bsa_fwd_phase_timers().
__device__ unsigned long long g_fwd_phase[64];
#define PT_FLUSH(base) PT_FLUSH_TO(g_fwd_phase, base)
#else
#define PT_FLUSH(base)
#endif

namespace bsa {

struct FwdParams {
  const int32_t* __restrict__ q2k_index;
  const int32_t* __restrict__ q2k_nums;
  const int32_t* __restrict__ block_sizes;
  const int32_t* __restrict__ work_order;
  const float* __restrict__ q_scale;
  const float* __restrict__ k_scale;
  const float* __restrict__ v_scale;
  uint8_t* out;  // 16-bit output, rows of D elements
  long long o_stride_b, o_stride_h, o_stride_s;  // bytes
  float* lse;
  float* partial_o;
  float* partial_lse;
  int* status;
  long long bs_stride_b, bs_stride_h;
  int fixed_count, cap;
  int B, Hq, Hkv, G, Hidx, packed;
  int Sq, Sk, NqT, Nkv;
  int D;  // head dimension (64, 96 or 128): narrower heads ride on the 128-wide tiles, the tensor maps zero-fill
  int splits;
  int f16;  // 16-bit inputs are IEEE half instead of bfloat16 (128-token blocks, unsplit only)
  int num_work;  // B * Hidx * NqT * splits
  float scale_log2;
};

constexpr int kThreads = 256;  // warps 6 and 7 only complete the second warpgroup (register re-balancing is per warpgroup)
constexpr int kSoftmaxThreads = 128;  // warps 0-3: one thread per query row
constexpr int kMmaWarp = 4;           // issues every MMA of the CTA
constexpr int kLoadWarp = 5;          // TMA producer
constexpr int kCtasPerSm = 2;

template <bool FP8>
struct FwdCfg {
  static constexpr int kElt = FP8 ? 1 : 2;
  static constexpr int kTileBytes = 128 * 128 * kElt;  // one Q / K / V tile
  static constexpr int kSlabs = FP8 ? 1 : 2;           // 128-byte-wide column slabs per tile
  static constexpr int kSlabBytes = 128 * 128;         // 128 rows x 128 B
  // One ring of K/V stages in consumption order K(0), V(0), K(1), V(1), ...  Two CTAs share an SM, so a CTA may
  // take half of its shared memory: Q + two stages for 16-bit inputs, Q + four stages for e4m3.
  static constexpr int kStages = FP8 ? 4 : 2;
  static constexpr int kMmaK = FP8 ? 32 : 16;
  static constexpr int kKSteps = 128 / kMmaK;
  static constexpr int kPColsPerStep = 8;  // tensor-memory columns of P per MMA k step
  // smem: Q | KV stages | 32 barriers | tmem base, abort flag
  static constexpr int kSmemBytes = kTileBytes + kStages * kTileBytes + 256 + 16;
};
// two CTAs (plus 1 KB each that the system reserves) must fit the 196 KB carve-out, which leaves the L1 60 KB
static_assert(kCtasPerSm * (FwdCfg<false>::kSmemBytes + 1024) <= 196 * 1024, "two CTAs per SM");

struct WorkItem {
  int b, hidx, m, split;
  int hkv, g;        // kv head and head offset inside the group (unpacked GQA)
  int count;         // live entries of the q2k row
  int it_begin, it_end;  // KV iterations of this split
  const int32_t* row;    // q2k row
};

template <int BLK>
__device__ __forceinline__ WorkItem decode_work(const FwdParams& p, int w) {
  WorkItem t;
  t.split = w % p.splits;
  int r = w / p.splits;
  if (p.work_order) {
    r = p.work_order[r];
    if (r < 0 || r >= p.B * p.Hidx * p.NqT) {  // a corrupt order must not turn into a wild access
      if (atomicCAS(p.status, 0, (int)kStatusBadIndex) == 0) p.status[2] = r;
      r = 0;
    }
  }
  t.m = r % p.NqT;
  r /= p.NqT;
  t.hidx = r % p.Hidx;
  t.b = r / p.Hidx;
  if (p.packed) {
    t.hkv = t.hidx;
    t.g = 0;
  } else {
    t.hkv = t.hidx / p.G;
    t.g = t.hidx % p.G;
  }
  const long long row_id = ((long long)t.b * p.Hidx + t.hidx) * p.NqT + t.m;
  int c = p.q2k_nums ? p.q2k_nums[row_id] : p.fixed_count;
  c = max(0, min(c, p.cap));
  t.count = c;
  t.row = p.q2k_index + row_id * p.cap;
  constexpr int kPerIt = 128 / BLK;
  const int n_it = (c + kPerIt - 1) / kPerIt;
  t.it_begin = (int)(((long long)n_it * t.split) / p.splits);
  t.it_end = (int)(((long long)n_it * (t.split + 1)) / p.splits);
  return t;
}

// Work item of this CTA in band `band` of the work list: bands are walked back and forth (CTA c takes
// c, 2G-1-c, 2G+c, ...), so that with a longest-first list every CTA gets a similar total.
__device__ __forceinline__ int snake_work(int band) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  return band * G + ((band & 1) ? (G - 1 - c) : c);
}

// Valid token count of KV block j for (b, h): min(block_sizes[j], tokens physically left), >= 0.
template <int BLK>
__device__ __forceinline__ int block_len(const FwdParams& p, int b, int h, int j) {
  if (j < 0 || j >= p.Nkv) return 0;
  int lim = min(BLK, p.Sk - j * BLK);
  if (p.block_sizes) {
    lim = min(lim, p.block_sizes[b * p.bs_stride_b + h * p.bs_stride_h + j]);
  }
  return max(lim, 0);
}

template <int BLK, bool FP8, bool SPLIT>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
bsa_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using Cfg = FwdCfg<FP8>;
  constexpr int NS = Cfg::kStages;
  // everything lives in dynamic shared memory (no static allocation), so the 1024-byte alignment the
  // swizzled tiles need comes from the declaration itself and no slack has to be reserved
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sQ = smem_raw;
  uint8_t* sKV = sQ + Cfg::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + NS * Cfg::kTileBytes);
  const uint32_t bar_base = smem_u32(bars);
  auto BAR = [&](int i) { return bar_base + (uint32_t)i * 8u; };
  constexpr int kQFull = 0, kQEmpty = 1, kKvFull = 2, kKvEmpty = 2 + NS, kSFull = 2 + 2 * NS, kPHalf = kSFull + 1,
                kPFull = kPHalf + 1, kOFinal = kPFull + 1, kNumBars = kOFinal + 1;
  static_assert(kNumBars <= 32, "barrier slots");
  uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(bars + 32);
  volatile int& s_abort = *reinterpret_cast<volatile int*>(bars + 33);
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // uniform over the CTA: nothing has been set up yet
    if (threadIdx.x == 0 && atomicCAS(p.status, 0, (int)kStatusBadIndex) == 0) p.status[2] = 999;
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  WaitCtx wctx{&s_abort, p.status};

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(BAR(kQFull), 1);
    mbar_init(BAR(kQEmpty), 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(BAR(kKvFull + i), 1);
      mbar_init(BAR(kKvEmpty + i), 1);
    }
    mbar_init(BAR(kSFull), 1);
    // every softmax thread arrives itself: measured faster than one elected arrival per warp
    mbar_init(BAR(kPHalf), kSoftmaxThreads);
    mbar_init(BAR(kPFull), kSoftmaxThreads);
    mbar_init(BAR(kOFinal), 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == kMmaWarp) {
    // half of the SM's tensor memory: the other half belongs to the CTA that shares the SM
    tmem_alloc(smem_u32(&s_tmem_base), 256);
    tmem_relinquish();
  }
  if (warp == kLoadWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const uint32_t tS = tmem, tO = tmem + 128u;  // S (fp32; P overwrites its head) and O, 128 columns each

  const int seq_per_tile = p.packed ? (BLK / p.G) : BLK;  // sequence positions covered by one q tile

  if (warp == kLoadWarp) {
    // ======================================= TMA producer =======================================
    setmaxnreg_dec<40>();
    uint32_t ring_cnt = 0, q_cnt = 0;
    bool ok = true;
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < p.num_work && ok; ++band) {
      const int w = snake_work(band);
      if (w >= p.num_work) continue;
      const WorkItem t = decode_work<BLK>(p, w);
      const int n_it = t.it_end - t.it_begin;
      if (n_it <= 0) continue;
      PT_MARK(0)
      ok = mbar_wait(BAR(kQEmpty), (q_cnt & 1) ^ 1, wctx, 100);
      if (!ok) break;
      PT_MARK(1)
      if (lane == 0) {
        // a 64-row query tile fills only the top half of each slab
        mbar_arrive_expect_tx(BAR(kQFull), Cfg::kSlabs * BLK * 128);
#pragma unroll
        for (int sl = 0; sl < Cfg::kSlabs; ++sl) {
          tma_load_5d(smem_u32(sQ + sl * Cfg::kSlabBytes), &tm_q, BAR(kQFull), sl * (128 / Cfg::kElt), t.g,
                      t.m * seq_per_tile, t.hkv, t.b);
        }
      }
      ++q_cnt;
      for (int i = 0; i < n_it && ok; ++i) {
        const int it = t.it_begin + i;
        int j0, j1;
        if (BLK == 128) {
          j0 = t.row[it];
          j1 = j0;
        } else {
          j0 = t.row[2 * it];
          j1 = (2 * it + 1 < t.count) ? t.row[2 * it + 1] : j0;
        }
#pragma unroll
        for (int which = 0; which < 2; ++which) {  // K(i), then V(i)
          const CUtensorMap* tm = which ? &tm_v : &tm_k;
          const uint32_t stage = ring_cnt % NS;
          PT_MARK(0)
          ok = mbar_wait(BAR(kKvEmpty + stage), ((ring_cnt / NS) & 1) ^ 1, wctx, 101);
          if (!ok) break;
          PT_MARK(2)
          if (lane == 0) {
            uint8_t* dst = sKV + stage * Cfg::kTileBytes;
            mbar_arrive_expect_tx(BAR(kKvFull + stage), Cfg::kTileBytes);
#pragma unroll
            for (int sl = 0; sl < Cfg::kSlabs; ++sl) {
              const int c0 = sl * (128 / Cfg::kElt);
              if (BLK == 128) {
                tma_load_4d(smem_u32(dst + sl * Cfg::kSlabBytes), tm, BAR(kKvFull + stage), c0, j0 * 128, t.hkv, t.b);
              } else {
                tma_load_4d(smem_u32(dst + sl * Cfg::kSlabBytes), tm, BAR(kKvFull + stage), c0, j0 * 64, t.hkv, t.b);
                tma_load_4d(smem_u32(dst + sl * Cfg::kSlabBytes + 64 * 128), tm, BAR(kKvFull + stage), c0, j1 * 64,
                            t.hkv, t.b);
              }
            }
          }
          ++ring_cnt;
        }
      }
    }
    PT_FLUSH(48)
  } else if (warp == kMmaWarp) {
    // ========================================= MMA issue ========================================
    // Order inside a tile: QK(0), {PV(0), QK(1)}, {PV(1), QK(2)}, ...: S(i+1) overwrites the tensor-memory
    // columns P(i) lives in, so it follows PV(i) in this thread's program order.  While this CTA's softmax works on
    // S(i), the tensor pipe belongs to the CTA that shares the SM.
    setmaxnreg_dec<40>();
    const uint32_t kFmt = (FP8 || p.f16) ? 0u : 1u;  // e4m3 (kind::f8f6f4) or f16 (kind::f16) = 0, bf16 = 1
    const uint32_t idesc_qk = umma_idesc(kFmt, kFmt, 0, 0, 128, 128);
    // Narrower heads (D = 64 or 96, 16-bit inputs only) use the head's own tile shape: QK^T contracts over D / 16
    // k steps (the tensor maps zero-fill the rest of the 128-wide shared-memory tiles, which is then never read) and
    // PV produces D output columns.
    const uint32_t idesc_pv = umma_idesc(kFmt, kFmt, 0, 1, 128, (uint32_t)p.D);
    const int qk_steps = FP8 ? Cfg::kKSteps : p.D / 16;
    const uint32_t led = lane == 0;
    // MMA steps of PV issued on the first release of P: half of the tile for 16-bit inputs, three quarters for e4m3
    constexpr int kPvFirst = FP8 ? 3 * Cfg::kKSteps / 4 : Cfg::kKSteps / 2;
    uint32_t ring_pos = 0, q_cnt = 0, p_cnt = 0;
    const uint64_t q_desc = umma_desc_sw128(smem_u32(sQ), 0, 1024);
    const uint64_t k_desc0 = umma_desc_sw128(smem_u32(sKV), 0, 1024);                                      // K-major view
    const uint64_t v_desc0 = umma_desc_sw128(smem_u32(sKV), FP8 ? 0u : (uint32_t)Cfg::kSlabBytes, 1024);  // MN-major
    bool ok = true;
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < p.num_work && ok; ++band) {
      const int w = snake_work(band);
      if (w >= p.num_work) continue;
      const WorkItem t = decode_work<BLK>(p, w);
      const int n_it = t.it_end - t.it_begin;
      if (n_it <= 0) continue;
      PT_MARK(0)
      ok = mbar_wait(BAR(kQFull), q_cnt & 1, wctx, 200);
      if (!ok) break;
      PT_MARK(1)
      ++q_cnt;
      auto issue_qk = [&](bool last) -> bool {
        const uint32_t stage = ring_pos % NS;
        PT_MARK(0)
        if (!mbar_wait(BAR(kKvFull + stage), (ring_pos / NS) & 1, wctx, 201)) return false;
        ++ring_pos;
        PT_MARK(2)
        tc_fence_after();
        const uint64_t kd = k_desc0 + (uint64_t)stage * (Cfg::kTileBytes >> 4);
#pragma unroll
        for (int k = 0; k < Cfg::kKSteps; ++k) {
          const uint64_t off = FP8 ? (uint64_t)(k * 2) : (uint64_t)((k >> 2) * (Cfg::kSlabBytes >> 4) + (k & 3) * 2);
          if (FP8) umma_f8_ss_led(tS, q_desc + off, kd + off, idesc_qk, k > 0, led);
          else umma_f16_ss_led(tS, q_desc + off, kd + off, idesc_qk, k > 0, (k < qk_steps) ? led : 0u);
        }
        umma_commit_led(BAR(kSFull), led);
        umma_commit_led(BAR(kKvEmpty + stage), led);
        if (last) umma_commit_led(BAR(kQEmpty), led);  // the tile's last S: Q may be replaced
        __syncwarp();
        PT_MARK(7)
        return true;
      };
      auto issue_pv = [&](int i, bool last) -> bool {
        const uint32_t stage = ring_pos % NS;
        PT_MARK(0)
        if (!mbar_wait(BAR(kKvFull + stage), (ring_pos / NS) & 1, wctx, 202)) return false;
        ++ring_pos;
        PT_MARK(3)
        if (!mbar_wait(BAR(kPHalf), p_cnt & 1, wctx, 203)) return false;  // first half of P
        PT_MARK(4)
        tc_fence_after();
        const uint64_t vd = v_desc0 + (uint64_t)stage * (Cfg::kTileBytes >> 4);
        auto pv_steps = [&](int k0, int k1) {
#pragma unroll
          for (int k = k0; k < k1; ++k) {
            // V is MN-major: one k step = kMmaK token rows of 128 B; the second 64-channel slab of a
            // bf16 tile is reached through the leading byte offset.
            const uint64_t db = vd + (uint64_t)(k * ((Cfg::kMmaK * 128) >> 4));
            const uint32_t a_t = tS + (uint32_t)k * Cfg::kPColsPerStep;
            if (FP8) umma_f8_ts_led(tO, a_t, db, idesc_pv, (i > 0) || (k > 0), led);
            else umma_f16_ts_led(tO, a_t, db, idesc_pv, (i > 0) || (k > 0), led);
          }
        };
        pv_steps(0, kPvFirst);
        PT_MARK(6)
        if (!mbar_wait(BAR(kPFull), p_cnt & 1, wctx, 204)) return false;  // second half
        PT_MARK(4)
        ++p_cnt;
        tc_fence_after();
        pv_steps(kPvFirst, Cfg::kKSteps);
        umma_commit_led(BAR(kKvEmpty + stage), led);
        if (last) umma_commit_led(BAR(kOFinal), led);
        __syncwarp();
        PT_MARK(6)
        return true;
      };
      ok = issue_qk(n_it == 1);
      for (int i = 0; i < n_it && ok; ++i) {
        ok = issue_pv(i, i == n_it - 1);
        if (ok && i + 1 < n_it) ok = issue_qk(i + 2 == n_it);
      }
    }
    PT_MARK(0)
    PT_FLUSH(32)
  } else if (warp < 4) {
    // ===================================== softmax + epilogue ===================================
    // Four warps, one thread per query row (= tensor-memory lane), all 128 score columns of the row.
    setmaxnreg_inc<216>();
    const int row = threadIdx.x;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const bool row_active = (BLK == 128) || (row < 64);  // warp-uniform
    uint32_t s_cnt = 0, of_cnt = 0;
    bool ok = true;
    const bool need_mask_meta = (p.block_sizes != nullptr) || (p.Sk % BLK != 0);
    constexpr float kRescaleThreshold = FP8 ? 1.8073549f /* log2(448/128) */ : 8.0f;
    constexpr float kPBias = FP8 ? 7.0f : 0.0f;
    PT_DECL

    for (int band = 0; band * (int)gridDim.x < p.num_work && ok; ++band) {
      const int w = snake_work(band);
      if (w >= p.num_work) continue;
      const WorkItem t = decode_work<BLK>(p, w);
      const int n_it = t.it_end - t.it_begin;
      float m_cur = -INFINITY;  // running max, log2 domain (scale applied)
      float l_sum = 0.f;        // running sum relative to m_cur

      // query row -> (sequence position, head)
      int seq, hq;
      if (p.packed) {
        seq = t.m * seq_per_tile + row / p.G;
        hq = t.hkv * p.G + row % p.G;
      } else {
        seq = t.m * BLK + row;
        hq = t.hidx;
      }
      const bool row_valid = row_active && (seq < p.Sq);
      float q_row_scale = 1.f;
      if (FP8) {
        q_row_scale = row_valid ? p.q_scale[((long long)t.b * p.Hq + hq) * p.Sq + seq] : 0.f;
      }

      for (int i = 0; i < n_it && ok; ++i) {
        // mask metadata for this KV iteration
        int len0 = BLK, len1 = BLK;
        int j0 = 0;
        int j1 = 0;
        if (need_mask_meta || FP8) {
          const int it = t.it_begin + i;
          if (BLK == 128) {
            j0 = t.row[it];
            len0 = block_len<BLK>(p, t.b, t.hkv, j0);
          } else {
            j0 = t.row[2 * it];
            len0 = block_len<BLK>(p, t.b, t.hkv, j0);
            const bool live1 = 2 * it + 1 < t.count;
            j1 = live1 ? t.row[2 * it + 1] : j0;
            len1 = live1 ? block_len<BLK>(p, t.b, t.hkv, j1) : 0;
          }
        } else if (BLK == 64) {
          const int it = t.it_begin + i;
          len1 = (2 * it + 1 < t.count) ? BLK : 0;
        }
        float ksc[8];
        if (FP8) {
          // eight 16-token scale groups of this 128-token tile: one 128-block, or four of each 64-block
          const int ngroups = (p.Sk + 15) / 16;
          const float* ks = p.k_scale + ((long long)t.b * p.Hkv + t.hkv) * ngroups;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int jb = (BLK == 128 || g < 4) ? j0 : j1;
            const int gi = (BLK == 128) ? jb * 8 + g : jb * 4 + (g & 3);
            ksc[g] = (jb >= 0 && jb < p.Nkv && gi < ngroups) ? ks[gi] * (q_row_scale * p.scale_log2) : 0.f;
          }
        }

        PT_MARK(0)
        ok = mbar_wait(BAR(kSFull), s_cnt & 1, wctx, 300);
        if (!ok) break;
        PT_MARK(1)
        ++s_cnt;
        tc_fence_after();
        if (!row_active) {
          // idle half of a 64-row tile: only the barrier protocol
          tc_fence_before();
          mbar_arrive(BAR(kPHalf));
          mbar_arrive(BAR(kPFull));
          continue;
        }
        float sv[128];
        uint32_t* su = reinterpret_cast<uint32_t*>(sv);
        const uint32_t t_row = tS + lane_base;
        const bool masked = (BLK == 128) ? (len0 < 128) : (len0 < 64 || len1 < 64);  // warp-uniform
        float bm;
        if (masked) {
          tmem_ld32(t_row + 0, su + 0);
          tmem_ld32(t_row + 32, su + 32);
          tmem_ld32(t_row + 64, su + 64);
          tmem_ld32(t_row + 96, su + 96);
          tmem_wait_ld();
          PT_MARK(2)
          if (masked) {
            if (BLK == 128) {
#pragma unroll
              for (int c = 0; c < 128; ++c) sv[c] = (c < len0) ? sv[c] : -INFINITY;
            } else {
#pragma unroll
              for (int c = 0; c < 64; ++c) sv[c] = (c < len0) ? sv[c] : -INFINITY;
#pragma unroll
              for (int c = 0; c < 64; ++c) sv[64 + c] = (c < len1) ? sv[64 + c] : -INFINITY;
            }
          }
          // ---- block max in the scaled log2 domain
          if (FP8) {
            bm = -INFINITY;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              float gm = sv[g * 16];
#pragma unroll
              for (int c = 1; c < 16; c += 2) gm = fmax3(gm, sv[g * 16 + c], sv[g * 16 + ((c + 1) & 15)]);
              // -inf * 0 would be NaN for fully masked groups beyond the sequence end
              const float scaled = (gm == -INFINITY) ? -INFINITY : gm * ksc[g];
              bm = fmaxf(bm, scaled);
            }
          } else {
            float m0 = sv[0], m1 = sv[1];
#pragma unroll
            for (int c = 2; c < 128; c += 4) {
              m0 = fmax3(m0, sv[c], sv[c + 1]);
              m1 = fmax3(m1, sv[(c + 2) & 127], sv[(c + 3) & 127]);
            }
            bm = fmaxf(m0, m1) * p.scale_log2;
          }
        } else if (FP8) {
          // common case, e4m3: group maxima (16 tokens share a K scale) of the first half while the second
          // half is still arriving
          tmem_ld32(t_row + 0, su + 0);
          tmem_ld32(t_row + 32, su + 32);
          tmem_wait_ld();
          tmem_ld32(t_row + 64, su + 64);
          tmem_ld32(t_row + 96, su + 96);
          bm = -INFINITY;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float gm = fmax3(sv[g * 16], sv[g * 16 + 1], sv[g * 16 + 2]);
#pragma unroll
            for (int c = 3; c < 15; c += 2) gm = fmax3(gm, sv[g * 16 + c], sv[g * 16 + c + 1]);
            gm = fmaxf(gm, sv[g * 16 + 15]);
            bm = fmaxf(bm, gm * ksc[g]);
          }
          tmem_wait_ld();
          PT_MARK(2)
#pragma unroll
          for (int g = 4; g < 8; ++g) {
            float gm = fmax3(sv[g * 16], sv[g * 16 + 1], sv[g * 16 + 2]);
#pragma unroll
            for (int c = 3; c < 15; c += 2) gm = fmax3(gm, sv[g * 16 + c], sv[g * 16 + c + 1]);
            gm = fmaxf(gm, sv[g * 16 + 15]);
            bm = fmaxf(bm, gm * ksc[g]);
          }
        } else {
          // common case: two 64-column halves; the second arrives while the maximum of the first is taken
          float m0, m1;
          tmem_ld32(t_row + 0, su + 0);
          tmem_ld32(t_row + 32, su + 32);
          tmem_wait_ld();
          tmem_ld32(t_row + 64, su + 64);
          tmem_ld32(t_row + 96, su + 96);
          m0 = fmax3(sv[0], sv[1], sv[2]);
          m1 = fmax3(sv[3], sv[4], sv[5]);
#pragma unroll
          for (int c = 6; c < 62; c += 4) {
            m0 = fmax3(m0, sv[c], sv[c + 1]);
            m1 = fmax3(m1, sv[c + 2], sv[c + 3]);
          }
          m0 = fmax3(m0, sv[62], sv[63]);
          tmem_wait_ld();
          PT_MARK(2)
#pragma unroll
          for (int c = 64; c < 128; c += 4) {
            m0 = fmax3(m0, sv[c], sv[c + 1]);
            m1 = fmax3(m1, sv[c + 2], sv[c + 3]);
          }
          bm = fmaxf(m0, m1) * p.scale_log2;
        }
        const float m_new = fmaxf(m_cur, bm);
        const bool first = (i == 0);
        if (first) {
          m_cur = m_new;
        } else {
          const bool need = (m_new - m_cur) > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            const float sc = (m_new == -INFINITY) ? 1.f : ex2_approx(m_cur - m_new);
            m_cur = m_new;
            l_sum *= sc;
            // rescale O in tensor memory (the previous PV has completed: the commit that signalled this S
            // was issued after it)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(tO + lane_base + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * sc);
              tmem_st32(tO + lane_base + c * 32, o);
            }
            tmem_wait_st();
          }
        }
        const float m_used = (m_cur == -INFINITY) ? 0.f : m_cur;
        const float neg_m = kPBias - m_used;
        PT_MARK(3)
        // ---- exponentials, row sum, P to tensor memory
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        if (FP8) {
          const uint64_t nm2 = pack2(neg_m, neg_m);
          if (masked) {
            // rare path (tail or shortened block): fp32 exponentials; masked columns hold -inf and a zero
            // scale there would make NaN, so they are selected explicitly
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t pk[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const int c = c4 * 32 + e * 4;
                const float sc = ksc[c >> 4];
                const float x0 = (sv[c] == -INFINITY) ? 0.f : ex2_approx(fmaf(sv[c], sc, neg_m));
                const float x1 = (sv[c + 1] == -INFINITY) ? 0.f : ex2_approx(fmaf(sv[c + 1], sc, neg_m));
                const float x2 = (sv[c + 2] == -INFINITY) ? 0.f : ex2_approx(fmaf(sv[c + 2], sc, neg_m));
                const float x3 = (sv[c + 3] == -INFINITY) ? 0.f : ex2_approx(fmaf(sv[c + 3], sc, neg_m));
                a0 += x0; a1 += x1; a2 += x2; a3 += x3;
                pk[e] = pack_e4m3x4(x0, x1, x2, x3);
              }
              if (c4 == 3) {
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(BAR(kPHalf));
              }
              tmem_st8(tS + lane_base + c4 * 8, pk);
            }
          } else {
            // The probabilities are rounded to e4m3 (three mantissa bits), so the exponentials are taken in
            // packed half precision: two results per special-function operation, one conversion to e4m3 per
            // pair.  The row sum runs in packed halves over at most 32 columns (four partial sums of four
            // terms, <= 4 * 448) and is flushed to fp32 per chunk.
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t pk[8];
              uint32_t hs[4];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const int c = c4 * 32 + e * 4;
                const float sc = ksc[c >> 4];
                const uint64_t sc2 = pack2(sc, sc);
                float x0, x1, x2, x3;
                unpack2(ffma2(pack2(sv[c], sv[c + 1]), sc2, nm2), x0, x1);
                unpack2(ffma2(pack2(sv[c + 2], sv[c + 3]), sc2, nm2), x2, x3);
                const uint32_t e01 = ex2_f16x2(pack_f16x2(x0, x1));
                const uint32_t e23 = ex2_f16x2(pack_f16x2(x2, x3));
                if (e < 2) {
                  hs[2 * e] = e01;
                  hs[2 * e + 1] = e23;
                } else {
                  hs[(2 * e) & 3] = hadd2(hs[(2 * e) & 3], e01);
                  hs[(2 * e + 1) & 3] = hadd2(hs[(2 * e + 1) & 3], e23);
                }
                pk[e] = pack_e4m3x4_f16(e01, e23);
              }
              float lo, hi;
              unpack_f16x2(hadd2(hadd2(hs[0], hs[1]), hadd2(hs[2], hs[3])), lo, hi);
              if (c4 & 1) { a2 += lo; a3 += hi; } else { a0 += lo; a1 += hi; }
              if (c4 == 3) {
                // the first three quarters of P (three of the four MMA k steps) are released on their own barrier
                // (a quarter later than for 16-bit inputs: measured 1.3 % faster), their stores long landed
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(BAR(kPHalf));
              }
              tmem_st8(tS + lane_base + c4 * 8, pk);
            }
          }
        } else {
          // the loop is instantiated once per 16-bit format so that the choice costs nothing per element
          auto exp_store = [&](auto is_f16) {
          const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2);
          const uint64_t nm2 = pack2(neg_m, neg_m);
          uint64_t s0 = pack2(0.f, 0.f), s1 = s0;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int c = c4 * 32 + e * 2;
              float x0, x1;
              unpack2(ffma2(pack2(sv[c], sv[c + 1]), sc2, nm2), x0, x1);
              x0 = ex2_approx(x0);
              x1 = ex2_approx(x1);
              if (e & 1) s1 = fadd2(s1, pack2(x0, x1));
              else s0 = fadd2(s0, pack2(x0, x1));
              pk[e] = decltype(is_f16)::value ? pack_f16x2(x0, x1) : pack_bf16x2(x0, x1);
            }
            if (c4 == 2) {
              // the first half of P (four MMA k steps) is released on its own barrier; waiting for its
              // stores only now, after the third chunk's arithmetic, keeps their latency off the path
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(BAR(kPHalf));
            }
            tmem_st16(tS + lane_base + c4 * 16, pk);
          }
          float y0, y1, y2, y3;
          unpack2(s0, y0, y1);
          unpack2(s1, y2, y3);
          a0 = y0; a1 = y1; a2 = y2; a3 = y3;
          };
          if (p.f16) exp_store(std::true_type{});
          else exp_store(std::false_type{});
        }
        l_sum += (a0 + a1) + (a2 + a3);
        PT_MARK(4)
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(BAR(kPFull));
        PT_MARK(5)
      }
      if (!ok) break;

      // ------------------------------------ tile epilogue ------------------------------------
      PT_MARK(0)
      const float inv = (l_sum > 0.f) ? (1.f / l_sum) : 0.f;
      const float lse_log2 = (l_sum > 0.f) ? (m_cur + lg2_approx(l_sum) - kPBias) : -INFINITY;
      if (n_it > 0) {
        ok = mbar_wait(BAR(kOFinal), of_cnt & 1, wctx, 310);
        if (!ok) break;
        ++of_cnt;
        tc_fence_after();
      }
      PT_MARK(6)
      // Every thread finalises its own row, 32 columns at a time, straight from tensor memory to global memory
      // (a row is 256 contiguous bytes).  The next tile's first PV overwrites O only after P(0) of that tile, which
      // these same threads write after this loop.
      const float* vs = FP8 ? p.v_scale + (long long)hq * 128 : nullptr;
      long long prow = 0;
      float4* dst_f = nullptr;
      uint4* dst_h = nullptr;
      if (SPLIT) {
        prow = (((long long)t.split * p.B + t.b) * p.Hq + hq) * p.Sq + seq;
        dst_f = reinterpret_cast<float4*>(p.partial_o + prow * 128);
      } else {
        dst_h = reinterpret_cast<uint4*>(p.out + (long long)t.b * p.o_stride_b + (long long)hq * p.o_stride_h +
                                         (long long)seq * p.o_stride_s);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float acc[32];
        if (row_active && n_it > 0) {
          uint32_t o[32];
          tmem_ld32(tO + lane_base + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) acc[e] = __uint_as_float(o[e]) * inv;
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) acc[e] = 0.f;
        }
        if (FP8) {
#pragma unroll
          for (int e = 0; e < 32; ++e) acc[e] *= vs[c * 32 + e];
        }
        if (row_valid) {
        if (SPLIT) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            dst_f[c * 8 + e] = make_float4(acc[4 * e], acc[4 * e + 1], acc[4 * e + 2], acc[4 * e + 3]);
        } else {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            if (c * 32 + ch * 8 < p.D) {  // narrower heads: the columns beyond D do not exist
              uint4 v;
              if (p.f16) {
                v.x = pack_f16x2(acc[ch * 8 + 0], acc[ch * 8 + 1]);
                v.y = pack_f16x2(acc[ch * 8 + 2], acc[ch * 8 + 3]);
                v.z = pack_f16x2(acc[ch * 8 + 4], acc[ch * 8 + 5]);
                v.w = pack_f16x2(acc[ch * 8 + 6], acc[ch * 8 + 7]);
              } else {
                v.x = pack_bf16x2(acc[ch * 8 + 0], acc[ch * 8 + 1]);
                v.y = pack_bf16x2(acc[ch * 8 + 2], acc[ch * 8 + 3]);
                v.z = pack_bf16x2(acc[ch * 8 + 4], acc[ch * 8 + 5]);
                v.w = pack_bf16x2(acc[ch * 8 + 6], acc[ch * 8 + 7]);
              }
              dst_h[c * 4 + ch] = v;
            }
          }
        }
        }
        __syncwarp();
      }
      tc_fence_before();
      if (row_valid) {
        if (SPLIT) p.partial_lse[prow] = lse_log2 * kLn2;
        else if (p.lse != nullptr) p.lse[((long long)t.b * p.Hq + hq) * p.Sq + seq] = lse_log2 * kLn2;
      }
      PT_MARK(7)
    }
    if (warp == 0) { PT_FLUSH(0) }
  } else {
    setmaxnreg_dec<40>();
  }

  // ------------------------------------------ teardown ------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// =================================================================================================
// host side
// =================================================================================================

template <int BLK, bool FP8, bool SPLIT>
static int launch_fwd(const bsa_fwd_args& a, const FwdParams& p, const CUtensorMap& tq,
                      const CUtensorMap& tk, const CUtensorMap& tv,
                      int num_sms, cudaStream_t stream) {
  using Cfg = FwdCfg<FP8>;
  auto kern = bsa_fwd_kernel<BLK, FP8, SPLIT>;
  {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "cudaFuncSetAttribute(smem): %s", cudaGetErrorString(e));
  }
  const int grid = p.num_work < kCtasPerSm * num_sms ? p.num_work : kCtasPerSm * num_sms;
  if (grid <= 0) return BSA_OK;
  kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "forward launch: %s", cudaGetErrorString(e));
  (void)a;
  return BSA_OK;
}

}  // namespace bsa

using namespace bsa;

#ifdef BSA_PHASE_TIMERS
// development builds only: copies the forward phase counters to the host and clears them
extern "C" int bsa_fwd_phase_timers(unsigned long long* host_out) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host_out, g_fwd_phase, sizeof(unsigned long long) * 64);
  static unsigned long long zeros[64];
  cudaMemcpyToSymbol(g_fwd_phase, zeros, sizeof(zeros));
  return 0;
}
#endif

extern "C" int bsa_fwd(const bsa_fwd_args* a, void* cuda_stream) {
  if (!a) return set_error(BSA_ERR_INVALID, "bsa_fwd: null args");
  if (a->blk != 64 && a->blk != 128) return set_error(BSA_ERR_INVALID, "bsa_fwd: blk must be 64 or 128");
  if (a->D != 128 && a->D != 96 && a->D != 64)
    return set_error(BSA_ERR_UNSUPPORTED, "bsa_fwd: head dimension %d not built (64, 96 or 128)", a->D);
  if (a->D != 128 && (a->blk != 128 || a->splits != 1 || a->dtype == BSA_DTYPE_E4M3))
    return set_error(BSA_ERR_UNSUPPORTED, "bsa_fwd: head dimensions below 128 are built for unsplit 16-bit 128-token blocks");
  if (a->dtype != BSA_DTYPE_BF16 && a->dtype != BSA_DTYPE_E4M3 && a->dtype != BSA_DTYPE_F16)
    return set_error(BSA_ERR_INVALID, "bsa_fwd: unknown dtype %d", a->dtype);
  if (a->dtype == BSA_DTYPE_F16 && (a->blk != 128 || a->splits != 1))
    return set_error(BSA_ERR_UNSUPPORTED, "bsa_fwd: float16 is built for unsplit 128-token blocks only");
  if (a->B < 1 || a->Hq < 1 || a->Hkv < 1 || a->Sq < 1 || a->Sk < 1)
    return set_error(BSA_ERR_INVALID, "bsa_fwd: non-positive extent");
  if (a->Hq % a->Hkv != 0) return set_error(BSA_ERR_INVALID, "bsa_fwd: Hq %% Hkv != 0");
  if (!a->q || !a->k || !a->v || !a->q2k_index || !a->status)
    return set_error(BSA_ERR_INVALID, "bsa_fwd: null tensor pointer");
  if (a->splits < 1 || a->splits > 256) return set_error(BSA_ERR_INVALID, "bsa_fwd: splits out of [1,256]");
  if (a->splits > 1 && (!a->partial_o || !a->partial_lse))
    return set_error(BSA_ERR_INVALID, "bsa_fwd: split run needs partial buffers");
  if (a->splits == 1) {
    // the output tensor map needs a 16-byte aligned base and 16-byte strides; checked here, before any CUDA call
    if (!a->out) return set_error(BSA_ERR_INVALID, "bsa_fwd: null out");
    if ((reinterpret_cast<uintptr_t>(a->out) & 15u) != 0)
      return set_error(BSA_ERR_INVALID, "out: base address must be 16-byte aligned");
    if ((a->o_stride[0] | a->o_stride[1] | a->o_stride[2]) % 8 != 0)
      return set_error(BSA_ERR_INVALID, "out: strides must be multiples of 8 elements");
  }
  if (a->cap < 0 || a->block_sparse_num < 0) return set_error(BSA_ERR_INVALID, "bsa_fwd: negative count");
  const bool fp8 = a->dtype == BSA_DTYPE_E4M3;
  const int G = a->Hq / a->Hkv;
  if (fp8 && (G != 1 || !a->q_scale || !a->k_scale || !a->v_scale))
    return set_error(BSA_ERR_INVALID, "bsa_fwd: FP8 path needs MHA and the three scale tensors");
  const int packed = a->pack_gqa != 0 && G > 1;
  if (packed && (a->blk % G) != 0) return set_error(BSA_ERR_INVALID, "bsa_fwd: pack_gqa needs blk %% group == 0");

  int dev = 0;
  cudaGetDevice(&dev);
  const int num_sms = bsa_num_sms(dev);
  if (num_sms <= 0) return set_error(BSA_ERR_CUDA, "bsa_fwd: cannot query the SM count");

  FwdParams p{};
  p.q2k_index = a->q2k_index;
  p.q2k_nums = a->q2k_nums;
  p.block_sizes = a->block_sizes;
  p.work_order = a->work_order;
  p.q_scale = a->q_scale;
  p.k_scale = a->k_scale;
  p.v_scale = a->v_scale;
  p.out = static_cast<uint8_t*>(a->out);
  p.o_stride_b = (long long)a->o_stride[0] * 2;
  p.o_stride_h = (long long)a->o_stride[1] * 2;
  p.o_stride_s = (long long)a->o_stride[2] * 2;
  p.lse = a->lse;
  p.partial_o = a->partial_o;
  p.partial_lse = a->partial_lse;
  p.status = a->status;
  p.bs_stride_b = a->bs_stride_b;
  p.bs_stride_h = a->bs_stride_h;
  p.fixed_count = a->block_sparse_num;
  p.cap = a->cap;
  p.B = a->B;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.G = G;
  p.packed = packed;
  p.Hidx = packed ? a->Hkv : a->Hq;
  p.Sq = a->Sq;
  p.Sk = a->Sk;
  const long long rows = packed ? (long long)a->Sq * G : a->Sq;
  p.NqT = (int)((rows + a->blk - 1) / a->blk);
  p.Nkv = (a->Sk + a->blk - 1) / a->blk;
  p.D = a->D;
  p.splits = a->splits;
  p.f16 = a->dtype == BSA_DTYPE_F16;
  const long long work = (long long)p.B * p.Hidx * p.NqT * p.splits;
  if (work > 0x7fffffffLL) return set_error(BSA_ERR_UNSUPPORTED, "bsa_fwd: more than 2^31 work items");
  p.num_work = (int)work;
  p.scale_log2 = a->softmax_scale * kLog2e;

  // tensor maps.  Q and O: 5-D (D, G, S, Hkv, B) so that a packed-GQA tile (blk/G sequence positions x G
  // heads) is one box; K and V: 4-D (D, S, Hkv, B).
  const int elt = fp8 ? 1 : 2;
  const CUtensorMapDataType dt16 = a->dtype == BSA_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : dt16;
  const uint32_t inner = 128 / elt;  // elements per 128-byte swizzle row
  CUtensorMap tq, tk, tv;
  {
    // the innermost extent is the true head dimension: boxes that reach beyond it read zeros / are clipped
    uint64_t dims[5] = {(uint64_t)a->D, (uint64_t)G, (uint64_t)a->Sq, (uint64_t)a->Hkv, (uint64_t)a->B};
    uint64_t str[4] = {(uint64_t)a->q_stride[1] * elt, (uint64_t)a->q_stride[2] * elt,
                       (uint64_t)a->q_stride[1] * G * elt, (uint64_t)a->q_stride[0] * elt};
    uint32_t box[5] = {inner, packed ? (uint32_t)G : 1u, (uint32_t)(packed ? a->blk / G : a->blk), 1, 1};
    int rc = make_tensor_map(&tq, dt, 5, a->q, dims, str, box, "q");
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)a->D, (uint64_t)a->Sk, (uint64_t)a->Hkv, (uint64_t)a->B};
    uint64_t kstr[3] = {(uint64_t)a->k_stride[2] * elt, (uint64_t)a->k_stride[1] * elt,
                        (uint64_t)a->k_stride[0] * elt};
    uint64_t vstr[3] = {(uint64_t)a->v_stride[2] * elt, (uint64_t)a->v_stride[1] * elt,
                        (uint64_t)a->v_stride[0] * elt};
    uint32_t box[4] = {inner, (uint32_t)a->blk, 1, 1};
    int rc = make_tensor_map(&tk, dt, 4, a->k, dims, kstr, box, "k");
    if (rc) return rc;
    rc = make_tensor_map(&tv, dt, 4, a->v, dims, vstr, box, "v");
    if (rc) return rc;
  }

  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  const bool split = a->splits > 1;
  if (fp8) {
    if (a->blk == 128)
      return split ? launch_fwd<128, true, true>(*a, p, tq, tk, tv, num_sms, stream)
                   : launch_fwd<128, true, false>(*a, p, tq, tk, tv, num_sms, stream);
    return split ? launch_fwd<64, true, true>(*a, p, tq, tk, tv, num_sms, stream)
                 : launch_fwd<64, true, false>(*a, p, tq, tk, tv, num_sms, stream);
  }
  if (a->blk == 128) {
    return split ? launch_fwd<128, false, true>(*a, p, tq, tk, tv, num_sms, stream)
                 : launch_fwd<128, false, false>(*a, p, tq, tk, tv, num_sms, stream);
  }
  return split ? launch_fwd<64, false, true>(*a, p, tq, tk, tv, num_sms, stream)
               : launch_fwd<64, false, false>(*a, p, tq, tk, tv, num_sms, stream);
}
