// Sparse-index construction on the device (integer work, HBM/latency bound):
//   block mask -> q2k index (ascending), q2k -> dense k2q (set semantics), q2k -> bucketed k2q CSR.
// All three are deterministic: every list comes out in ascending order, whatever the launch timing.
//
// Semantics: utils/block_sparse_index.py:20-129 (k2q: bitmap scatter + pack, zero padding),
// csrc/bwd/bucketed_k2q_csr.py:114-238 and its CPU model tests/test_bucketed_k2q_csr.py:12-74
// (one edge per occurrence, ids outside [0,Nkv) dropped, counts clamped to [0,cap], offsets running
// across the query groups of one (batch, head)).
#include "bsa_b200.h"
#include "bsa_common.cuh"
#include "bsa_host.h"

namespace bsa {

// ------------------------------------------------------------------------------------------------
// mask -> q2k: one warp per (b, h, q-block) row
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
mask_to_q2k_kernel(const uint8_t* __restrict__ mask, int32_t* __restrict__ index,
                   int32_t* __restrict__ nums, long long rows, int Nkv, int cap) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint8_t* mrow = mask + row * Nkv;
  int32_t* irow = index + row * cap;
  int found = 0;
  for (int c0 = 0; c0 < Nkv; c0 += 32) {
    const int c = c0 + lane;
    const bool on = (c < Nkv) && (mrow[c] != 0);
    const unsigned bal = __ballot_sync(0xffffffffu, on);
    const int pos = found + __popc(bal & ((1u << lane) - 1u));
    if (on && pos < cap) irow[pos] = c;
    found += __popc(bal);
  }
  const int n = min(found, cap);
  for (int c = n + lane; c < cap; c += 32) irow[c] = 0;
  if (lane == 0) nums[row] = n;
}

// ------------------------------------------------------------------------------------------------
// q2k -> dense k2q (set semantics).  The output itself serves as the flag matrix: zero it, scatter a
// 1 at [kv][q] for every live edge, then compact each [kv] row in place into ascending q ids.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ int live_count(const int32_t* nums, long long row, int fixed, int cap) {
  int c = nums ? nums[row] : fixed;
  return max(0, min(c, cap));
}

__global__ void __launch_bounds__(256)
k2q_scatter_kernel(const int32_t* __restrict__ q2k, const int32_t* __restrict__ nums, int fixed,
                   long long q_rows, int Nq, int cap, int Nkv, int32_t* __restrict__ k2q) {
  // one warp per q row
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= q_rows) return;
  const int lane = threadIdx.x & 31;
  const int cnt = live_count(nums, row, fixed, cap);
  const long long bh = row / Nq;
  const int q = (int)(row % Nq);
  for (int i = lane; i < cnt; i += 32) {
    const int kv = q2k[row * cap + i];
    if (kv >= 0 && kv < Nkv) k2q[(bh * Nkv + kv) * Nq + q] = 1;
  }
}

__global__ void __launch_bounds__(256)
k2q_compact_kernel(int32_t* __restrict__ k2q, int32_t* __restrict__ k2q_nums, long long kv_rows, int Nq) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= kv_rows) return;
  const int lane = threadIdx.x & 31;
  int32_t* r = k2q + row * Nq;
  int found = 0;
  for (int c0 = 0; c0 < Nq; c0 += 32) {
    const int c = c0 + lane;
    const bool on = (c < Nq) && (r[c] != 0);
    const unsigned bal = __ballot_sync(0xffffffffu, on);  // every flag of the chunk is read before any write
    const int pos = found + __popc(bal & ((1u << lane) - 1u));
    if (on) r[pos] = c;  // pos <= c: never ahead of the read cursor
    found += __popc(bal);
  }
  __syncwarp();
  for (int c = found + lane; c < Nq; c += 32) r[c] = 0;
  if (lane == 0) k2q_nums[row] = found;
}

// ------------------------------------------------------------------------------------------------
// bucketed k2q CSR
//   1. count   : offsets[b,h,g,kv] += 1 per edge (the array is zeroed first)
//   2. scan    : per (b,h) exclusive prefix over (g, kv), offsets[b,h,g,Nkv] = end of group g
//   3. scatter : position = atomicAdd(&offsets[b,h,g,kv], 1); afterwards offsets[..kv] holds the END of
//                row kv, i.e. the array is shifted by one entry
//   4. unshift : offsets[b,h,g,kv] = (kv == 0 ? group base : shifted[kv-1])
//   5. sort    : every CSR row ascending (this is what makes the result independent of atomics order)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
csr_count_kernel(const int32_t* __restrict__ q2k, const int32_t* __restrict__ nums, int fixed,
                 long long q_rows, int Nq, int cap, int Nkv, int bucket, int G,
                 int32_t* __restrict__ offsets) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= q_rows) return;
  const int lane = threadIdx.x & 31;
  const int cnt = live_count(nums, row, fixed, cap);
  const long long bh = row / Nq;
  const int q = (int)(row % Nq);
  const int g = q / bucket;
  int32_t* base = offsets + (bh * G + g) * (long long)(Nkv + 1);
  for (int i = lane; i < cnt; i += 32) {
    const int kv = q2k[row * cap + i];
    if (kv >= 0 && kv < Nkv) atomicAdd(base + kv, 1);
  }
}

// one block per (b,h): exclusive scan over G * (Nkv+1) slots where slot Nkv of each group holds 0 on entry
__global__ void __launch_bounds__(1024)
csr_scan_kernel(int32_t* __restrict__ offsets, int G, int Nkv) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  int32_t* base = offsets + (long long)blockIdx.x * G * (Nkv + 1);
  const int total = G * (Nkv + 1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < total; c0 += 1024) {
    const int i = c0 + threadIdx.x;
    const int v = (i < total) ? base[i] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    const int excl = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + x - v;
    if (i < total) base[i] = excl;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_sums[31];
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
csr_scatter_kernel(const int32_t* __restrict__ q2k, const int32_t* __restrict__ nums, int fixed,
                   long long q_rows, int Nq, int cap, int Nkv, int bucket, int G,
                   int32_t* __restrict__ offsets, int32_t* __restrict__ indices, long long idx_cap) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= q_rows) return;
  const int lane = threadIdx.x & 31;
  const int cnt = live_count(nums, row, fixed, cap);
  const long long bh = row / Nq;
  const int q = (int)(row % Nq);
  const int g = q / bucket;
  int32_t* base = offsets + (bh * G + g) * (long long)(Nkv + 1);
  int32_t* out = indices + bh * idx_cap;
  for (int i = lane; i < cnt; i += 32) {
    const int kv = q2k[row * cap + i];
    if (kv >= 0 && kv < Nkv) {
      const int pos = atomicAdd(base + kv, 1);
      if (pos >= 0 && pos < idx_cap) out[pos] = q;
    }
  }
}

// one block per (b,h,g): undo the shift left by the cursor atomics
__global__ void __launch_bounds__(256)
csr_unshift_kernel(int32_t* __restrict__ offsets, int G, int Nkv) {
  const long long bhg = blockIdx.x;
  const int g = (int)(bhg % G);
  int32_t* base = offsets + bhg * (long long)(Nkv + 1);
  const int group_base = (g == 0) ? 0 : base[-1];  // slot Nkv of the previous group: never a cursor
  // walk from the top so that a slot is read before the chunk below overwrites it
  for (int hi = Nkv - 1; hi >= 0; hi -= 256) {
    const int i = hi - (int)threadIdx.x;
    int v = 0;
    if (i >= 0) v = (i == 0) ? group_base : base[i - 1];
    __syncthreads();
    if (i >= 0) base[i] = v;
    __syncthreads();
  }
}

constexpr int kSortSmemInts = 1024;       // per warp: 1024 entries of a short row, or 4096 byte counters
constexpr int kSortCountRange = 4 * kSortSmemInts;
constexpr int kSortRankMax = 64;          // rows up to this length are rank-sorted (n^2 / 32 steps per lane)

// One warp per CSR row: ascending order, in place.  Every entry of a row of query group g is a query block of
// that group, i.e. lies in [g * bucket, g * bucket + bucket): rows longer than kSortRankMax are therefore
// sorted by counting (one byte counter per query block of the group in shared memory, O(n + bucket) work, any
// row length) as long as the group has at most kSortCountRange query blocks - which covers every default
// bucket (384 / 512 / 1088 / 1152).  Short rows are rank-sorted.  What is left (a caller-chosen bucket above
// 4096 blocks, or a query block listed more than 255 times in one row) takes a rank sort up to 1024 entries
// and an odd-even transposition sort in global memory beyond.
__global__ void __launch_bounds__(128)
csr_sort_kernel(const int32_t* __restrict__ offsets, int32_t* __restrict__ indices, long long n_rows,
                int G, int Nkv, int Nq, int bucket, long long idx_cap) {
  __shared__ int32_t buf[4][kSortSmemInts];
  const long long r = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  // r enumerates (bh, g, kv)
  const int kv = (int)(r % Nkv);
  const long long bhg = r / Nkv;
  const long long bh = bhg / G;
  const int g = (int)(bhg % G);
  const int32_t* off = offsets + bhg * (long long)(Nkv + 1);
  const int beg = off[kv], end = off[kv + 1];
  const int n = end - beg;
  if (n <= 1) return;
  int32_t* row = indices + bh * idx_cap + beg;
  const int q_lo = g * bucket;
  const int range = min(bucket, Nq - q_lo);
  bool counted = false;
  if (n > kSortRankMax && range <= kSortCountRange) {
    uint32_t* cnt = reinterpret_cast<uint32_t*>(buf[w]);
    const int words = (range + 3) >> 2;
    for (int i = lane; i < words; i += 32) cnt[i] = 0;
    __syncwarp();
    bool overflow = false;
    for (int i = lane; i < n; i += 32) {
      const int q = row[i] - q_lo;
      if (q < 0 || q >= range) {  // cannot happen for rows written by the scatter pass; never index outside
        overflow = true;
        continue;
      }
      const uint32_t sh = 8u * (uint32_t)(q & 3);
      const uint32_t old = atomicAdd(cnt + (q >> 2), 1u << sh);
      overflow |= ((old >> sh) & 0xffu) == 0xffu;
    }
    overflow = __any_sync(0xffffffffu, overflow);
    __syncwarp();
    if (!overflow) {
      // lane l owns the counters of words [l * wpl, (l + 1) * wpl): its share of the output starts at the
      // exclusive prefix of the lanes below
      const int wpl = (words + 31) >> 5;
      const int w0 = lane * wpl, w1 = min(words, w0 + wpl);
      int mine = 0;
      for (int j = w0; j < w1; ++j) {
        const uint32_t c = cnt[j];
        mine += (int)((c & 0xffu) + ((c >> 8) & 0xffu) + ((c >> 16) & 0xffu) + (c >> 24));
      }
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
      }
      int pos = incl - mine;
      for (int j = w0; j < w1; ++j) {
        uint32_t c = cnt[j];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          for (int k = (int)(c & 0xffu); k > 0; --k) row[pos++] = q_lo + 4 * j + b;
          c >>= 8;
        }
      }
      counted = true;
    }
  }
  if (counted) return;
  if (n <= kSortSmemInts) {
    for (int i = lane; i < n; i += 32) buf[w][i] = row[i];
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
      const int v = buf[w][i];
      int rank = 0;
      for (int j = 0; j < n; ++j) {
        const int u = buf[w][j];
        rank += (u < v) || (u == v && j < i);
      }
      row[rank] = v;
    }
  } else {
    for (int phase = 0; phase < n; ++phase) {
      for (int i = (phase & 1) + 2 * lane; i + 1 < n; i += 64) {
        const int a = row[i], b = row[i + 1];
        if (a > b) {
          row[i] = b;
          row[i + 1] = a;
        }
      }
      __syncwarp();
    }
  }
}

// ------------------------------------------------------------------------------------------------
// longest-first work order: stable counting sort of the rows by descending live count.
//   hist layout: [(cap - count) * chunks + chunk], chunks of 1024 consecutive rows, so that one exclusive
//   scan over the whole array yields, for every (count, chunk), the first output slot of that chunk's
//   rows with that count.  Stability keeps rows of one (batch, head) adjacent inside a count class.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
lpt_hist_kernel(const int32_t* __restrict__ nums, int rows, int cap, int chunks, int32_t* __restrict__ hist) {
  const int chunk = blockIdx.x;
  const int r = chunk * 1024 + threadIdx.x;
  if (r < rows) {
    const int c = max(0, min(nums[r], cap));
    atomicAdd(hist + (long long)(cap - c) * chunks + chunk, 1);
  }
}

__global__ void __launch_bounds__(1024)
lpt_scan_kernel(int32_t* __restrict__ hist, long long total) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (long long c0 = 0; c0 < total; c0 += 1024) {
    const long long i = c0 + threadIdx.x;
    const int v = (i < total) ? hist[i] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    if (i < total) hist[i] = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + x - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_sums[31];
    __syncthreads();
  }
}

__global__ void __launch_bounds__(1024)
lpt_scatter_kernel(const int32_t* __restrict__ nums, int rows, int cap, int chunks, const int32_t* __restrict__ hist,
                   int32_t* __restrict__ order) {
  __shared__ int16_t s_cnt[1024];
  const int chunk = blockIdx.x;
  const int r = chunk * 1024 + threadIdx.x;
  const int c = (r < rows) ? max(0, min(nums[r], cap)) : -1;
  s_cnt[threadIdx.x] = (int16_t)c;
  __syncthreads();
  if (r < rows) {
    int rank = 0;  // rows of this chunk with the same count and a smaller index
    for (int j = 0; j < (int)threadIdx.x; ++j) rank += (s_cnt[j] == (int16_t)c);
    const int pos = hist[(long long)(cap - c) * chunks + chunk] + rank;
    if (pos >= 0 && pos < rows) order[pos] = r;
  }
}

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return BSA_OK;
}

}  // namespace bsa

using namespace bsa;

extern "C" int bsa_mask_to_q2k(const uint8_t* mask, int32_t* index, int32_t* nums, int32_t B, int32_t H,
                               int32_t Nq, int32_t Nkv, int32_t cap, void* cuda_stream) {
  if (!mask || !index || !nums) return set_error(BSA_ERR_INVALID, "bsa_mask_to_q2k: null pointer");
  if (B < 1 || H < 1 || Nq < 1 || Nkv < 1 || cap < 1) return set_error(BSA_ERR_INVALID, "bsa_mask_to_q2k: non-positive extent");
  const long long rows = (long long)B * H * Nq;
  const long long blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return set_error(BSA_ERR_UNSUPPORTED, "bsa_mask_to_q2k: too many rows");
  mask_to_q2k_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(mask, index, nums, rows,
                                                                                               Nkv, cap);
  return check_launch("mask_to_q2k");
}

extern "C" int bsa_q2k_to_k2q(const int32_t* q2k_index, const int32_t* q2k_nums, int32_t block_sparse_num,
                              int32_t B, int32_t H, int32_t Nq, int32_t cap, int32_t Nkv, int32_t* k2q_index,
                              int32_t* k2q_nums, void* cuda_stream) {
  if (!k2q_index || !k2q_nums) return set_error(BSA_ERR_INVALID, "bsa_q2k_to_k2q: null output");
  if (B < 1 || H < 1 || Nq < 1 || Nkv < 1 || cap < 0) return set_error(BSA_ERR_INVALID, "bsa_q2k_to_k2q: bad extent");
  if (cap > 0 && !q2k_index) return set_error(BSA_ERR_INVALID, "bsa_q2k_to_k2q: null index");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  const long long q_rows = (long long)B * H * Nq;
  const long long kv_rows = (long long)B * H * Nkv;
  cudaError_t e = cudaMemsetAsync(k2q_index, 0, sizeof(int32_t) * kv_rows * Nq, st);
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_q2k_to_k2q memset: %s", cudaGetErrorString(e));
  if (cap > 0) {
    k2q_scatter_kernel<<<(unsigned)((q_rows + 7) / 8), 256, 0, st>>>(q2k_index, q2k_nums, block_sparse_num, q_rows, Nq,
                                                                    cap, Nkv, k2q_index);
    int rc = check_launch("k2q_scatter");
    if (rc) return rc;
  }
  k2q_compact_kernel<<<(unsigned)((kv_rows + 7) / 8), 256, 0, st>>>(k2q_index, k2q_nums, kv_rows, Nq);
  return check_launch("k2q_compact");
}

extern "C" int bsa_build_k2q_csr(const int32_t* q2k_index, const int32_t* q2k_nums, int32_t block_sparse_num,
                                 int32_t B, int32_t H, int32_t Nq, int32_t cap, int32_t Nkv,
                                 int32_t bucket_size_blocks, int32_t* offsets, int32_t* indices,
                                 void* cuda_stream) {
  if (!offsets || !indices) return set_error(BSA_ERR_INVALID, "bsa_build_k2q_csr: null output");
  if (B < 1 || H < 1 || Nq < 1 || Nkv < 1 || cap < 0 || bucket_size_blocks < 1)
    return set_error(BSA_ERR_INVALID, "bsa_build_k2q_csr: bad extent");
  if (cap > 0 && !q2k_index) return set_error(BSA_ERR_INVALID, "bsa_build_k2q_csr: null index");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int G = (Nq + bucket_size_blocks - 1) / bucket_size_blocks;
  const long long q_rows = (long long)B * H * Nq;
  const long long idx_cap = (long long)Nq * cap > 1 ? (long long)Nq * cap : 1;
  const long long n_off = (long long)B * H * G * (Nkv + 1);
  cudaError_t e = cudaMemsetAsync(offsets, 0, sizeof(int32_t) * n_off, st);
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_build_k2q_csr memset: %s", cudaGetErrorString(e));
  int rc;
  if (cap > 0) {
    csr_count_kernel<<<(unsigned)((q_rows + 7) / 8), 256, 0, st>>>(q2k_index, q2k_nums, block_sparse_num, q_rows, Nq,
                                                                  cap, Nkv, bucket_size_blocks, G, offsets);
    if ((rc = check_launch("csr_count"))) return rc;
  }
  csr_scan_kernel<<<(unsigned)(B * H), 1024, 0, st>>>(offsets, G, Nkv);
  if ((rc = check_launch("csr_scan"))) return rc;
  if (cap > 0) {
    csr_scatter_kernel<<<(unsigned)((q_rows + 7) / 8), 256, 0, st>>>(q2k_index, q2k_nums, block_sparse_num, q_rows,
                                                                    Nq, cap, Nkv, bucket_size_blocks, G, offsets,
                                                                    indices, idx_cap);
    if ((rc = check_launch("csr_scatter"))) return rc;
    csr_unshift_kernel<<<(unsigned)((long long)B * H * G), 256, 0, st>>>(offsets, G, Nkv);
    if ((rc = check_launch("csr_unshift"))) return rc;
    const long long n_rows = (long long)B * H * G * Nkv;
    csr_sort_kernel<<<(unsigned)((n_rows + 3) / 4), 128, 0, st>>>(offsets, indices, n_rows, G, Nkv, Nq,
                                                                   bucket_size_blocks, idx_cap);
    if ((rc = check_launch("csr_sort"))) return rc;
  }
  return BSA_OK;
}

extern "C" int64_t bsa_lpt_order_scratch_ints(int32_t rows, int32_t cap) {
  if (rows < 1 || cap < 0) return 0;
  return (int64_t)(cap + 1) * ((rows + 1023) / 1024);
}

extern "C" int bsa_lpt_order(const int32_t* q2k_nums, int32_t rows, int32_t cap, int32_t* order, int32_t* scratch,
                             void* cuda_stream) {
  if (!q2k_nums || !order || !scratch) return set_error(BSA_ERR_INVALID, "bsa_lpt_order: null pointer");
  if (rows < 1 || cap < 0 || cap > 32000) return set_error(BSA_ERR_INVALID, "bsa_lpt_order: bad extent");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int chunks = (rows + 1023) / 1024;
  const long long total = (long long)(cap + 1) * chunks;
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int32_t) * total, st);
  if (e != cudaSuccess) return set_error(BSA_ERR_CUDA, "bsa_lpt_order memset: %s", cudaGetErrorString(e));
  int rc;
  lpt_hist_kernel<<<chunks, 1024, 0, st>>>(q2k_nums, rows, cap, chunks, scratch);
  if ((rc = check_launch("lpt_hist"))) return rc;
  lpt_scan_kernel<<<1, 1024, 0, st>>>(scratch, total);
  if ((rc = check_launch("lpt_scan"))) return rc;
  lpt_scatter_kernel<<<chunks, 1024, 0, st>>>(q2k_nums, rows, cap, chunks, scratch, order);
  return check_launch("lpt_scatter");
}
