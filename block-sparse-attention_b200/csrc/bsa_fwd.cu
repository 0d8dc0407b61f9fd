// Block-sparse attention forward for sm_100a: TMA gathers of the K/V blocks named by the q2k index,
// tcgen05 QK^T and PV MMAs accumulating in tensor memory, online softmax with LSE.
//
// One persistent CTA per SM walks (q tile, split) work items.  Warp roles:
//   warps 0-3   softmax group 0: owns stream 0 (KV iterations 0, 2, 4, ...), one thread per query row
//   warps 4-7   softmax group 1: owns stream 1 (KV iterations 1, 3, 5, ...)
//   warps 8-9   MMA issue, one warp (one lane) per stream
//   warps 10-11 TMA producers, one warp (one lane) per stream; producer 0 also loads the Q tiles
// The four non-softmax warps give registers up (setmaxnreg) in favour of the softmax groups.
// Tensor memory (512 columns): S0 @0, S1 @128, O0 @256, O1 @384 (fp32, 128 lanes x 128 columns each);
// the probabilities P_s overwrite the head of S_s (bf16: 64 columns, e4m3: 32 columns) and are the
// A operand of the PV MMA straight from tensor memory.  The two streams keep independent running
// (max, sum, O) and are merged once per tile in the epilogue.
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

constexpr int kThreads = 384;
constexpr int kSoftmaxThreads = 256;
constexpr int kMmaWarp = 8;
constexpr int kLoadWarp = 10;  // warps 8 and 9 issue the MMAs of stream 0 and 1, warps 10 and 11 load their K/V tiles


template <bool FP8>
struct FwdCfg {
  static constexpr int kElt = FP8 ? 1 : 2;
  static constexpr int kTileBytes = 128 * 128 * kElt;  // one Q / K / V tile
  static constexpr int kSlabs = FP8 ? 1 : 2;           // 128-byte-wide column slabs per tile
  static constexpr int kSlabBytes = 128 * 128;         // 128 rows x 128 B
  static constexpr int kStages = 4;
  // each stream owns a private ring of K/V stages (stream 0 the first kRing0 stages), consumed strictly in
  // order by that stream's issuing warp: a parity wait is then never more than one phase behind.
  // Two stages per stream (the K and the V tile of one iteration) measured faster than deeper rings on every
  // workload (cfg2 3.54 -> 3.42 ms against 3 + 2 stages; e4m3 1.64 -> 1.61 ms against 4 + 4)
  static constexpr int kRing0 = 2;
  static constexpr int kOBytes = 128 * 128 * 2;  // bf16 output staging
  static constexpr int kMmaK = FP8 ? 32 : 16;
  static constexpr int kKSteps = 128 / kMmaK;
  static constexpr int kPColsPerStep = FP8 ? 8 : 8;  // tensor-memory columns of P per MMA k step
  // smem: Q | O | KV stages | 32 barriers | stats [2][128] float2 | tmem base, abort flag | 2 turn barriers
  static constexpr int kSmemBytes = kTileBytes + kOBytes + kStages * kTileBytes + 256 + 2048 + 16 + 16;
};

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
__global__ void __launch_bounds__(kThreads, 1)
bsa_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const FwdParams p) {
  using Cfg = FwdCfg<FP8>;
  constexpr int NS = Cfg::kStages;
  // everything lives in dynamic shared memory (no static allocation), so the 1024-byte alignment the
  // swizzled tiles need comes from the declaration itself and no slack has to be reserved
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sO = sQ + Cfg::kTileBytes;
  uint8_t* sKV = sO + Cfg::kOBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + NS * Cfg::kTileBytes);
  // barrier slots
  //  0: q_full  1: q_empty  2..2+NS: kv_full  2+NS..2+2NS: kv_empty
  //  then s_full[2], p_full[2], o_final
  const uint32_t bar_base = smem_u32(bars);
  auto BAR = [&](int i) { return bar_base + (uint32_t)i * 8u; };
  constexpr int kQFull = 0, kQEmpty = 1, kKvFull = 2, kKvEmpty = 2 + NS, kSFull = 2 + 2 * NS,
                kPFull = kSFull + 2, kOFinal = kPFull + 2, kEpiA = kOFinal + 2, kGrpB = kEpiA + 1,
                kPHalf = kGrpB + 2, kNumBars = kPHalf + 2;
  float2 (*s_stats)[128] = reinterpret_cast<float2 (*)[128]>(bars + 32);  // [2][128] (max, sum)
  uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(bars + 32 + 256);
  volatile int& s_abort = *reinterpret_cast<volatile int*>(bars + 32 + 256 + 1);
  const uint32_t turn_base = smem_u32(bars + 32 + 256 + 2);  // two more barriers: the issuers' turn tokens
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
    mbar_init(BAR(kQEmpty), 2);
    for (int i = 0; i < NS; ++i) {
      mbar_init(BAR(kKvFull + i), 1);
      mbar_init(BAR(kKvEmpty + i), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(kSFull + s), 1);
      // every softmax thread arrives itself: measured faster than one elected arrival per warp
      mbar_init(BAR(kPFull + s), 128);
      mbar_init(BAR(kPHalf + s), 128);
    }
    mbar_init(turn_base, 1);
    mbar_init(turn_base + 8, 1);
    mbar_init(BAR(kOFinal), 1);  // one per stream: a stream without work in a tile neither arrives nor is waited for
    mbar_init(BAR(kOFinal + 1), 1);
    mbar_init(BAR(kEpiA), kSoftmaxThreads);
    mbar_init(BAR(kGrpB), kSoftmaxThreads);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  static_assert(kNumBars <= 32, "barrier slots");
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&s_tmem_base), 512);
    tmem_relinquish();
  }
  if (warp == kLoadWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    if (!SPLIT) tma_prefetch_desc(&tm_o);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const uint32_t tS[2] = {tmem + 0u, tmem + 128u};
  const uint32_t tO[2] = {tmem + 256u, tmem + 384u};

  const int seq_per_tile = p.packed ? (BLK / p.G) : BLK;  // sequence positions covered by one q tile

  if (warp == kLoadWarp || warp == kLoadWarp + 1) {
    // ======================================= TMA producers ======================================
    // One producer warp per stream: each fills only its own stream's ring, so a full ring of one stream
    // never holds back the loads of the other.  Producer 0 also loads the Q tiles.
    setmaxnreg_dec<56>();
    const int ls = warp - kLoadWarp;
    uint32_t ring_cnt[2] = {0, 0};  // tiles produced so far into each stream's ring
    uint32_t q_cnt = 0;
    bool ok = true;
    PT_DECL
    for (int band = 0; band * (int)gridDim.x < p.num_work && ok; ++band) {
      const int w = snake_work(band);
      if (w >= p.num_work) continue;
      const WorkItem t = decode_work<BLK>(p, w);
      const int n_it = t.it_end - t.it_begin;
      if (n_it <= 0) continue;
      PT_MARK(0)
      if (ls == 0) {
        // Q tile
        ok = mbar_wait(BAR(kQEmpty), (q_cnt & 1) ^ 1, wctx, 100);
        if (!ok) break;
        PT_MARK(1)
        if (lane == 0) {
          // a 64-row query tile fills only the top half of each slab
          mbar_arrive_expect_tx(BAR(kQFull), Cfg::kSlabs * BLK * 128);
#pragma unroll
          for (int sl = 0; sl < Cfg::kSlabs; ++sl) {
            tma_load_5d(smem_u32(sQ + sl * Cfg::kSlabBytes), &tm_q, BAR(kQFull), sl * (128 / Cfg::kElt),
                        t.g, t.m * seq_per_tile, t.hkv, t.b);
          }
        }
        ++q_cnt;
      }

      // K/V tiles of this producer's stream in its consumption order: K(s), V(s), K(s+2), V(s+2), ...
      auto issue_tile = [&](const CUtensorMap* tm, int strm, int blk0, int blk1) -> bool {
        const uint32_t depth = strm ? (uint32_t)(NS - Cfg::kRing0) : (uint32_t)Cfg::kRing0;
        const uint32_t stage = (strm ? (uint32_t)Cfg::kRing0 : 0u) + ring_cnt[strm] % depth;
        const uint32_t ph = (ring_cnt[strm] / depth) & 1;
        PT_MARK(0)
        if (!mbar_wait(BAR(kKvEmpty + stage), ph ^ 1, wctx, 101)) return false;
        PT_MARK(2)
        if (lane == 0) {
          uint8_t* dst = sKV + stage * Cfg::kTileBytes;
          mbar_arrive_expect_tx(BAR(kKvFull + stage), Cfg::kTileBytes);
#pragma unroll
          for (int sl = 0; sl < Cfg::kSlabs; ++sl) {
            const int c0 = sl * (128 / Cfg::kElt);
            if (BLK == 128) {
              tma_load_4d(smem_u32(dst + sl * Cfg::kSlabBytes), tm, BAR(kKvFull + stage), c0,
                          blk0 * 128, t.hkv, t.b);
            } else {
              tma_load_4d(smem_u32(dst + sl * Cfg::kSlabBytes), tm, BAR(kKvFull + stage), c0,
                          blk0 * 64, t.hkv, t.b);
              tma_load_4d(smem_u32(dst + sl * Cfg::kSlabBytes + 64 * 128), tm, BAR(kKvFull + stage),
                          c0, blk1 * 64, t.hkv, t.b);
            }
          }
        }
        ++ring_cnt[strm];
        return true;
      };
      // block ids of KV iteration `it` (relative to the row start)
      auto fetch = [&](int it, int& j0, int& j1) {
        if (BLK == 128) {
          j0 = t.row[it];
          j1 = j0;
        } else {
          j0 = t.row[2 * it];
          j1 = (2 * it + 1 < t.count) ? t.row[2 * it + 1] : j0;
        }
      };
      for (int i = ls; i < n_it && ok; i += 2) {
        int j0, j1;
        fetch(t.it_begin + i, j0, j1);
        ok = issue_tile(&tm_k, ls, j0, j1);
        if (ok) ok = issue_tile(&tm_v, ls, j0, j1);
      }
    }
    PT_FLUSH(48)
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ========================================= MMA issue ========================================
    // One issuing warp per stream.  tcgen05.mma issue stalls the issuing thread at the execution rate,
    // so with a single issuer the tensor pipe idles during every barrier wait and commit; with two
    // issuers one stream's bookkeeping overlaps the other stream's MMAs.  Per stream the order
    // PV(i) -> QK(i+2) is program order of one thread, which is what the aliasing of P_s with S_s needs.
    // The two issuers take turns: QK(0), QK(1), {PV(0),QK(2)}, {PV(1),QK(3)}, ... enter the tensor pipe
    // as whole batches in iteration order.  Left to themselves the streams lock in phase (both in their
    // softmax, then both in their MMAs, measured); batches handed over by a token keep them half a
    // cycle apart, so one stream's softmax runs under the other stream's MMAs.
    setmaxnreg_dec<56>();
    const int s = warp - kMmaWarp;
    const uint32_t tS_s = tmem + 128u * (uint32_t)s, tO_s = tmem + 256u + 128u * (uint32_t)s;
    const uint32_t kFmt = (FP8 || p.f16) ? 0u : 1u;  // e4m3 (kind::f8f6f4) or f16 (kind::f16) = 0, bf16 = 1
    const uint32_t idesc_qk = umma_idesc(kFmt, kFmt, 0, 0, 128, 128);
    // Narrower heads (D = 64 or 96, 16-bit inputs only) use the head's own tile shape: QK^T contracts over D / 16
    // k steps (the tensor maps zero-fill the rest of the 128-wide shared-memory tiles, which is then never read) and
    // PV produces D output columns.
    const uint32_t idesc_pv = umma_idesc(kFmt, kFmt, 0, 1, 128, (uint32_t)p.D);
    const int qk_steps = FP8 ? Cfg::kKSteps : p.D / 16;
    uint32_t ring_pos = 0, q_cnt = 0, p_cnt = 0;  // ring_pos: tiles of this stream's ring consumed so far
    const uint32_t ring_depth = s ? (uint32_t)(NS - Cfg::kRing0) : (uint32_t)Cfg::kRing0;
    const uint32_t ring_first = s ? (uint32_t)Cfg::kRing0 : 0u;
    bool ok = true;
    uint32_t turn_cnt = 0;      // completed waits on this issuer's turn barrier
    auto turn_wait = [&]() -> bool {
      const bool r = mbar_wait(turn_base + 8u * s, turn_cnt & 1, wctx, 205);
      ++turn_cnt;
      return r;
    };
    auto turn_pass = [&]() {
      if (lane == 0) mbar_arrive(turn_base + 8u * (s ^ 1));
      __syncwarp();
    };
    // descriptors are built once; a byte offset b inside a tile is an addition of b >> 4 to the low word
    const uint64_t q_desc = umma_desc_sw128(smem_u32(sQ), 0, 1024);
    const uint64_t k_desc0 = umma_desc_sw128(smem_u32(sKV), 0, 1024);                               // K-major view
    const uint64_t v_desc0 = umma_desc_sw128(smem_u32(sKV), FP8 ? 0u : (uint32_t)Cfg::kSlabBytes, 1024);  // MN-major
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
      // this stream's ring holds K(s), V(s), K(s+2), V(s+2), ... and is consumed in exactly that order
      auto issue_qk = [&](int i, bool take_turn) -> bool {
        const uint32_t stage = ring_first + ring_pos % ring_depth;
        PT_MARK(0)
        if (!mbar_wait(BAR(kKvFull + stage), (ring_pos / ring_depth) & 1, wctx, 201)) return false;
        ++ring_pos;
        PT_MARK(2)
        if (take_turn && !turn_wait()) return false;
        PT_MARK(5)
        PT_MARK(0)
        {
          const uint32_t led = lane == 0;
          const uint64_t kd = k_desc0 + (uint64_t)stage * (Cfg::kTileBytes >> 4);
#pragma unroll
          for (int k = 0; k < Cfg::kKSteps; ++k) {
            const uint64_t off = FP8 ? (uint64_t)(k * 2) : (uint64_t)((k >> 2) * (Cfg::kSlabBytes >> 4) + (k & 3) * 2);
            if (FP8) umma_f8_ss_led(tS_s, q_desc + off, kd + off, idesc_qk, k > 0, led);
            else umma_f16_ss_led(tS_s, q_desc + off, kd + off, idesc_qk, k > 0, (k < qk_steps) ? led : 0u);
          }
          umma_commit_led(BAR(kSFull + s), led);
          umma_commit_led(BAR(kKvEmpty + stage), led);
        }
        PT_MARK(7)
        return true;
      };
      auto issue_pv = [&](int i, bool take_turn) -> bool {
        const uint32_t stage = ring_first + ring_pos % ring_depth;
        PT_MARK(0)
        if (!mbar_wait(BAR(kKvFull + stage), (ring_pos / ring_depth) & 1, wctx, 202)) return false;
        ++ring_pos;
        PT_MARK(3)
        if (!mbar_wait(BAR(kPHalf + s), p_cnt & 1, wctx, 203)) return false;  // first half of P_s
        PT_MARK(4)
        if (take_turn && !turn_wait()) return false;
        PT_MARK(5)
        tc_fence_after();
        const uint64_t vd = v_desc0 + (uint64_t)stage * (Cfg::kTileBytes >> 4);
        auto pv_steps = [&](int k0, int k1) {
#pragma unroll
          for (int k = k0; k < k1; ++k) {
            // V is MN-major: one k step = kMmaK token rows of 128 B; the second 64-channel slab of a
            // bf16 tile is reached through the leading byte offset.
            const uint64_t db = vd + (uint64_t)(k * ((Cfg::kMmaK * 128) >> 4));
            const uint32_t a_t = tS_s + (uint32_t)k * Cfg::kPColsPerStep;
            if (FP8) umma_f8_ts_led(tO_s, a_t, db, idesc_pv, (i >= 2) || (k > 0), lane == 0);
            else umma_f16_ts_led(tO_s, a_t, db, idesc_pv, (i >= 2) || (k > 0), lane == 0);
          }
        };
        PT_MARK(0)
        pv_steps(0, Cfg::kKSteps / 2);
        PT_MARK(6)
        PT_MARK(0)
        if (!mbar_wait(BAR(kPFull + s), p_cnt & 1, wctx, 204)) return false;  // second half
        PT_MARK(4)
        ++p_cnt;
        tc_fence_after();
        PT_MARK(0)
        pv_steps(Cfg::kKSteps / 2, Cfg::kKSteps);
        umma_commit_led(BAR(kKvEmpty + stage), lane == 0);
        PT_MARK(6)
        return true;
      };

      // turns of this tile: QK(0) [stream 0], QK(1) [stream 1], then batch i = {PV(i), QK(i+2)} by stream
      // i & 1.  Every turn but the first waits for the token of its predecessor and every turn but the last
      // passes it on, so all passes are consumed inside the tile (tiles are ordered among themselves by the
      // Q buffer: the next Q tile is loaded only after both issuers have finished this one).  Short rows
      // are not worth the hand-offs: below kTurnMinIters iterations the issuers run freely.
      constexpr int kTurnMinIters = 6;
      const bool turns = n_it >= kTurnMinIters;
      if (s == 0) {
        ok = issue_qk(0, false);
        if (ok && turns) turn_pass();
      } else if (n_it >= 2) {
        ok = issue_qk(1, turns);
        if (ok && turns) turn_pass();
      }
      for (int i = s; i < n_it && ok; i += 2) {
        ok = issue_pv(i, turns);
        if (ok && i + 2 < n_it) ok = issue_qk(i + 2, false);
        if (ok && turns && i + 1 < n_it) turn_pass();
      }
      if (!ok) break;
      // Q is free once the QK MMAs of BOTH streams have completed: each issuer signals for its own MMAs
      // (a stream without work arrives directly; it cannot arrive twice in one phase because the next Q
      // tile, which it waits for first, is only loaded after this phase has completed).  O_s is final
      // when stream s's own PV MMAs have completed.
      if (lane == 0) {
        if (s < n_it) {
          umma_commit(BAR(kQEmpty));
          umma_commit(BAR(kOFinal + s));
        } else {
          mbar_arrive(BAR(kQEmpty));
        }
      }
      __syncwarp();
    }
    PT_MARK(0)
    if (s == 0) { PT_FLUSH(32) } else { PT_FLUSH(40) }
  } else if (warp < 8) {
    // ===================================== softmax + epilogue ===================================
    setmaxnreg_inc<216>();
    const int grp = warp >> 2;                 // stream owned by this group
    const int row = threadIdx.x & 127;         // query row inside the tile = tensor-memory lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const bool row_active = (BLK == 128) || (row < 64);  // warp-uniform
    uint32_t s_cnt = 0, of_cnt[2] = {0, 0}, epi_a = 0, grp_b = 0;
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

      for (int i = grp; i < n_it && ok; i += 2) {
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
        ok = mbar_wait(BAR(kSFull + grp), s_cnt & 1, wctx, 300 + grp);
        if (!ok) break;
        PT_MARK(1)
        ++s_cnt;
        tc_fence_after();
        if (!row_active) {
          // idle half of a 64-row tile: only the barrier protocol
          tc_fence_before();
          mbar_arrive(BAR(kPHalf + grp));
          mbar_arrive(BAR(kPFull + grp));
          continue;
        }
        float sv[128];
        uint32_t* su = reinterpret_cast<uint32_t*>(sv);
        const uint32_t t_row = tS[grp] + lane_base;
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
        const bool first = (i == grp);
        if (first) {
          m_cur = m_new;
        } else {
          const bool need = (m_new - m_cur) > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            const float sc = (m_new == -INFINITY) ? 1.f : ex2_approx(m_cur - m_new);
            m_cur = m_new;
            l_sum *= sc;
            // rescale O_s in tensor memory (the previous PV of this stream has completed: the commit
            // that signalled S_s was issued after it)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(tO[grp] + lane_base + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * sc);
              tmem_st32(tO[grp] + lane_base + c * 32, o);
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
              if (c4 == 2) {
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(BAR(kPHalf + grp));
              }
              tmem_st8(tS[grp] + lane_base + c4 * 8, pk);
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
              if (c4 == 2) {
                // first half of P_s (two MMA k steps) released on its own barrier, its stores long landed
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(BAR(kPHalf + grp));
              }
              tmem_st8(tS[grp] + lane_base + c4 * 8, pk);
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
              // the first half of P_s (four MMA k steps) is released on its own barrier; waiting for its
              // stores only now, after the third chunk's arithmetic, keeps their latency off the path
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(BAR(kPHalf + grp));
            }
            tmem_st16(tS[grp] + lane_base + c4 * 16, pk);
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
        mbar_arrive(BAR(kPFull + grp));
        PT_MARK(5)
      }
      if (!ok) break;

      // ------------------------------------ tile epilogue ------------------------------------
      PT_MARK(0)
      // The (max, sum) pairs of the two streams are exchanged while the last PV MMAs are still running.
      // The same rendezvous orders this tile's staging writes after the previous tile's output store.
      s_stats[grp][row] = make_float2(m_cur, l_sum);
      if (!SPLIT && (threadIdx.x & 127) == 0) tma_store_wait_read<0>();
      ok = mbar_rendezvous_poll(BAR(kEpiA), epi_a, wctx, 320);
      if (!ok) break;
      const float2 st0 = s_stats[0][row];
      const float2 st1 = s_stats[1][row];
      const float m_all = fmaxf(st0.x, st1.x);
      const float w0 = (st0.x == -INFINITY) ? 0.f : ex2_approx(st0.x - m_all);
      const float w1 = (st1.x == -INFINITY) ? 0.f : ex2_approx(st1.x - m_all);
      const float denom = st0.y * w0 + st1.y * w1;
      const float inv = (denom > 0.f) ? (1.f / denom) : 0.f;
      const float f0 = w0 * inv, f1 = w1 * inv;
      const bool has0 = n_it > 0, has1 = n_it > 1;
      if (n_it > 0) {
        ok = mbar_wait(BAR(kOFinal), of_cnt[0] & 1, wctx, 310 + grp);
        if (!ok) break;
        ++of_cnt[0];
        if (n_it > 1) {
          ok = mbar_wait(BAR(kOFinal + 1), of_cnt[1] & 1, wctx, 312 + grp);
          if (!ok) break;
          ++of_cnt[1];
        }
        tc_fence_after();
      }
      PT_MARK(6)

      // this group finalises output columns [64*grp, 64*grp+64)
      float acc[64];
#pragma unroll
      for (int e = 0; e < 64; ++e) acc[e] = 0.f;
      if (row_active) {
        if (has0) {
          uint32_t o[64];
          tmem_ld32(tO[0] + lane_base + grp * 64, o);
          tmem_ld32(tO[0] + lane_base + grp * 64 + 32, o + 32);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 64; ++e) acc[e] = __uint_as_float(o[e]) * f0;
        }
        if (has1) {
          uint32_t o[64];
          tmem_ld32(tO[1] + lane_base + grp * 64, o);
          tmem_ld32(tO[1] + lane_base + grp * 64 + 32, o + 32);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 64; ++e) acc[e] = fmaf(__uint_as_float(o[e]), f1, acc[e]);
        }
      }
      tc_fence_before();

      if (FP8) {
        const float* vs = p.v_scale + (long long)hq * 128 + grp * 64;
#pragma unroll
        for (int e = 0; e < 64; ++e) acc[e] *= vs[e];
      }
      const float lse_log2 = (denom > 0.f) ? (m_all + lg2_approx(denom) - kPBias) : -INFINITY;

      if (SPLIT) {
        if (row_valid) {
          const long long prow = (((long long)t.split * p.B + t.b) * p.Hq + hq) * p.Sq + seq;
          float4* dst = reinterpret_cast<float4*>(p.partial_o + prow * 128 + grp * 64);
#pragma unroll
          for (int e = 0; e < 16; ++e)
            dst[e] = make_float4(acc[4 * e], acc[4 * e + 1], acc[4 * e + 2], acc[4 * e + 3]);
          if (grp == 0) p.partial_lse[prow] = lse_log2 * kLn2;
        }
        // every thread has read its share of O0 / O1: the next tile may overwrite them
        ok = mbar_rendezvous_poll(BAR(kGrpB), grp_b, wctx, 323);
        if (!ok) break;
      } else {
        // stage bf16 in shared memory in the 128-byte-swizzled layout the output tensor map expects
        const bool issuer = (threadIdx.x & 127) == 0;
        if (row_active) {
          uint8_t* slab = sO + grp * (128 * 128);
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
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
            *reinterpret_cast<uint4*>(slab + row * 128 + ((ch ^ (row & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        // both groups: the staging tile is complete, and every thread has read its share of O0 / O1, so the
        // next tile may overwrite them
        ok = mbar_rendezvous_poll(BAR(kGrpB), grp_b, wctx, 323);
        if (!ok) break;
        if (issuer && grp * 64 < p.D) {  // a 64-wide head has no second column slab to store
          const int cs = t.m * seq_per_tile;
          tma_store_5d(&tm_o, smem_u32(sO + grp * (128 * 128)), grp * 64, t.g, cs, t.hkv, t.b);
          tma_store_commit();
        }
        if (grp == 0 && row_valid && p.lse != nullptr) {
          p.lse[((long long)t.b * p.Hq + hq) * p.Sq + seq] = lse_log2 * kLn2;
        }
      }
      PT_MARK(7)
    }
    if ((threadIdx.x & 127) == 0 && !SPLIT) tma_store_wait_all<0>();
    if ((warp & 3) == 0) { PT_FLUSH(grp * 8) }
  } else {
    setmaxnreg_dec<56>();
  }

  // ------------------------------------------ teardown ------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// =================================================================================================
// host side
// =================================================================================================

template <int BLK, bool FP8, bool SPLIT>
static int launch_fwd(const bsa_fwd_args& a, const FwdParams& p, const CUtensorMap& tq,
                      const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                      int num_sms, cudaStream_t stream) {
  using Cfg = FwdCfg<FP8>;
  auto kern = bsa_fwd_kernel<BLK, FP8, SPLIT>;
  {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "cudaFuncSetAttribute(smem): %s", cudaGetErrorString(e));
  }
  const int grid = p.num_work < num_sms ? p.num_work : num_sms;
  if (grid <= 0) return BSA_OK;
  kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, to, p);
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
  CUtensorMap tq, tk, tv, to;
  {
    // the innermost extent is the true head dimension: boxes that reach beyond it read zeros / are clipped
    uint64_t dims[5] = {(uint64_t)a->D, (uint64_t)G, (uint64_t)a->Sq, (uint64_t)a->Hkv, (uint64_t)a->B};
    uint64_t str[4] = {(uint64_t)a->q_stride[1] * elt, (uint64_t)a->q_stride[2] * elt,
                       (uint64_t)a->q_stride[1] * G * elt, (uint64_t)a->q_stride[0] * elt};
    uint32_t box[5] = {inner, packed ? (uint32_t)G : 1u, (uint32_t)(packed ? a->blk / G : a->blk), 1, 1};
    int rc = make_tensor_map(&tq, dt, 5, a->q, dims, str, box, "q");
    if (rc) return rc;
    if (a->splits == 1) {
      uint64_t ostr[4] = {(uint64_t)a->o_stride[1] * 2, (uint64_t)a->o_stride[2] * 2,
                          (uint64_t)a->o_stride[1] * G * 2, (uint64_t)a->o_stride[0] * 2};
      uint32_t obox[5] = {64, packed ? (uint32_t)G : 1u, (uint32_t)(packed ? a->blk / G : a->blk), 1, 1};
      rc = make_tensor_map(&to, dt16, 5, a->out, dims, ostr, obox, "out");
      if (rc) return rc;
    } else {
      to = tq;
    }
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
      return split ? launch_fwd<128, true, true>(*a, p, tq, tk, tv, to, num_sms, stream)
                   : launch_fwd<128, true, false>(*a, p, tq, tk, tv, to, num_sms, stream);
    return split ? launch_fwd<64, true, true>(*a, p, tq, tk, tv, to, num_sms, stream)
                 : launch_fwd<64, true, false>(*a, p, tq, tk, tv, to, num_sms, stream);
  }
  if (a->blk == 128) {
    return split ? launch_fwd<128, false, true>(*a, p, tq, tk, tv, to, num_sms, stream)
                 : launch_fwd<128, false, false>(*a, p, tq, tk, tv, to, num_sms, stream);
  }
  return split ? launch_fwd<64, false, true>(*a, p, tq, tk, tv, to, num_sms, stream)
               : launch_fwd<64, false, false>(*a, p, tq, tk, tv, to, num_sms, stream);
}
