/*
 * libbsa_b200.so — C ABI of the B200-native (sm_100a) block-sparse attention engine.
 *
 * This is the boundary a maintainer of NVIDIA-JerryChen/Block-Sparse-Attention binds in place of the
 * compiled CuTe-DSL callables (JIT or AOT) that bsa_attn_interface.py launches today.  Every entry
 * point is asynchronous on the given CUDA stream, allocates nothing, and takes only device pointers,
 * sizes and element strides.  Return value: 0 = launched, negative = argument rejected before any
 * launch (bsa_last_error() gives the text).  Device-side trouble (a bounded wait that expired) is
 * reported through the caller's `status` buffer (int32[4], zeroed by the caller; word 0 != 0 means
 * the results of that launch are invalid).
 *
 * Path references are relative to the reference repository.
 */
#ifndef BSA_B200_H_
#define BSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSA_B200_ABI_VERSION 1

enum bsa_dtype { BSA_DTYPE_BF16 = 0, BSA_DTYPE_E4M3 = 1, BSA_DTYPE_F16 = 2 /* unsplit 128-token blocks only */ };

/* Error codes returned by the entry points (negative). */
enum bsa_error {
  BSA_OK = 0,
  BSA_ERR_INVALID = -1,     /* argument validation failed                        */
  BSA_ERR_UNSUPPORTED = -2, /* shape/dtype combination not built (e.g. D != 128) */
  BSA_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed                 */
  BSA_ERR_WORKSPACE = -4    /* caller-supplied workspace too small               */
};

/* Library identification. */
int bsa_abi_version(void);
/* Text of the last error raised on the calling thread (never NULL). */
const char* bsa_last_error(void);
/* Number of SMs of `device` (148 on B200); the persistent grids are sized from it. */
int bsa_num_sms(int device);
/*
 * Self-test of the bounded device-side wait (no counterpart in the reference, whose waits are unbounded:
 * csrc/fwd/sm100_blk64/bsa_fwd_helpers.py:41-86).  Launches one small CTA whose two warps wait, with a
 * budget of `limit_ns` nanoseconds (at most 1 s), on an mbarrier that nothing arrives at - the same wait
 * routine every role of the attention kernels uses.  When the budget runs out the kernel writes
 * status[0..3] = {1, block, site 900 or 901, thread}, leaves through the common exit and sets *returned = 1.
 * Nothing faults and the context stays usable; `status` is int32[4], zeroed by the caller, `returned` int32[1].
 */
int bsa_selftest_wait(uint64_t limit_ns, int32_t* status, int32_t* returned, void* cuda_stream);

/*
 * Forward attention over the KV blocks selected by q2k_block_index.
 *
 * Replaces the compiled callables of
 *   bsa_attn_interface.py:3706-3718   (BF16 blk128: fn(q,k,v,out,lse,scale,index,block_sizes,num,nums,stream))
 *   bsa_attn_interface.py:2765-2781   (blk64, BF16 and Sage FP8, optional split producer)
 *   bsa_attn_interface.py:3336-3344   (Sage FP8 blk128, 14-argument form)
 * i.e. the kernels csrc/fwd/sm100_blk128/bsa_fwd_sm100.py, csrc/fwd/sm100_blk64/bsa_fwd_sm100.py and
 * csrc/fwd/sm100_blk128/bsa_fwd_sm100_fp8_fused_pv.py.
 *
 * Layouts (strides in elements, innermost dimension contiguous):
 *   q   [B, Hq,  Sq, D]   k, v [B, Hkv, Sk, D]   out [B, Hq, Sq, D] bf16
 *   lse [B, Hq, Sq] f32 contiguous, natural log, scale included; may be NULL
 *   q2k_index [B, Hidx, Nq, cap] int32 contiguous; only the first `count` entries of a row are read
 *   q2k_nums  [B, Hidx, Nq] int32 contiguous or NULL (then count = block_sparse_num for every row)
 *   block_sizes: NULL, or int32 with element strides (bs_stride_b, bs_stride_h, 1) over [B, H, Nkv]
 *                (stride 0 = broadcast), valid tokens of each KV block
 * Hidx = Hkv and Nq = ceil(Sq*G/blk) when pack_gqa != 0 (G = Hq/Hkv, packed row r = seq*G + head
 * offset), else Hidx = Hq and Nq = ceil(Sq/blk).
 *
 * splits > 1: every (q tile, split) writes a normalised FP32 partial to partial_o
 * [splits, B, Hq, Sq, D] and its log-sum-exp to partial_lse [splits, B, Hq, Sq]; `out`/`lse` are not
 * touched and the caller runs bsa_fwd_combine afterwards.
 *
 * D = 128; with 16-bit inputs, 128-token blocks and splits = 1 also D = 64 and 96, the head dimensions of the
 * reference's 128-token forward (csrc/fwd/sm100_blk128/bsa_fwd_sm100.py:75-78).
 *
 * work_order: the persistent CTAs walk the tile rows in this order (CTA c takes entries c, 2G-1-c, 2G+c, ...
 * of it, G = grid size); a longest-first order balances skewed per-row counts.  NULL = natural order.
 *
 * dtype = BSA_DTYPE_E4M3 selects the Sage FP8 path: q, k, v hold e4m3 bytes, q_scale [B,H,Sq],
 * k_scale [B,H,ceil(Sk/16)] and v_scale [H,D] are the multiplicative dequantisation factors
 * (contiguous f32), Hq must equal Hkv.
 */
typedef struct bsa_fwd_args {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  const int32_t* q2k_index;
  const int32_t* q2k_nums;
  const int32_t* block_sizes;
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  float* partial_o;
  float* partial_lse;
  const int32_t* work_order; /* NULL, or a permutation of the B*Hidx*Nq tile rows (see bsa_lpt_order) */
  int32_t* status;
  int64_t q_stride[3]; /* batch, head, seq */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int64_t bs_stride_b;
  int64_t bs_stride_h;
  int32_t dtype; /* enum bsa_dtype */
  int32_t blk;   /* 64 or 128 */
  int32_t B, Hq, Hkv, Sq, Sk, D;
  int32_t cap;              /* last extent of q2k_index */
  int32_t block_sparse_num; /* used when q2k_nums == NULL */
  int32_t pack_gqa;
  int32_t splits; /* >= 1 */
  float softmax_scale;
  int32_t reserved;
} bsa_fwd_args;

int bsa_fwd(const bsa_fwd_args* args, void* cuda_stream);

/*
 * LSE-weighted merge of split-KV partials: lse = log sum_s exp(lse_s), out = sum_s exp(lse_s - lse) O_s.
 * Rows whose partial LSEs are all -inf give out = 0, lse = -inf.
 * Replaces the 10-argument combine callable of bsa_attn_interface.py:1944-1955
 * (csrc/fwd/sm100_blk64/bsa_fwd_combine.py).
 *   partial_o [splits, rows, D] f32, partial_lse [splits, rows] f32, rows = B*Hq*Sq in BHS order;
 *   out bf16 addressed with o_stride (batch, head, seq); lse [rows] f32 or NULL.
 */
int bsa_fwd_combine(const float* partial_o, const float* partial_lse, void* out, float* lse,
                    int32_t splits, int32_t B, int32_t H, int32_t Sq, int32_t D,
                    const int64_t o_stride[3], void* cuda_stream);

/*
 * Sage FP8 quantiser: per-token Q scale (BF16-rounded reciprocal and product), per-16-token scale of the
 * mean-centred K, per-(head, channel) V scale shared over batch and sequence; e4m3 outputs.
 * Replaces the three Triton kernels of bsa_fp8_quant.py:10-104 launched by quantize_sage_bhsd (:122-218).
 * All tensors contiguous BHSD with D = 128.  k_mean [B,H,128] f32 and partials
 * [2, B, H, ceil(Sk/1024), 128] f32 are caller-supplied scratch (size from bsa_quantize_sage_scratch_floats).
 */
int bsa_quantize_sage(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8,
                      float* q_scale, float* k_scale, float* v_scale, float* k_mean, float* partials,
                      int32_t B, int32_t H, int32_t Sq, int32_t Sk, void* cuda_stream);
int64_t bsa_quantize_sage_scratch_floats(int32_t B, int32_t H, int32_t Sk);

/*
 * Same quantiser for callers that cannot provide scratch memory (this entry point has no counterpart in
 * the reference).  Think of a server whose memory pool is frozen after start-up, or a plain C host
 * without a device allocator of its own: the K mean and the chunk statistics are kept in a 4 MiB array
 * that is part of the library image (each GPU that loads the library holds it until the process ends).
 * Nothing is allocated or freed, here or in anything it calls.
 *   limit   : B*H*(1 + 2*ceil(Sk/1024))*128 floats <= BSA_QUANTIZE_STATIC_SCRATCH_FLOATS (1 Mi);
 *             larger problems are rejected with BSA_ERR_WORKSPACE and must use bsa_quantize_sage.
 *   set-up  : the first call on each device looks the array's device address up; make that first call
 *             outside any stream capture.  Host threads may make it concurrently: the per-device slot is an
 *             atomic, and every thread that finds it empty stores the same address.
 *   sharing : all calls on a device use the same array.  Calls that can overlap on the GPU (different
 *             streams without ordering) race on it; serialise them.  No state has to be cleared between
 *             calls: every value read is written earlier in the same call.
 */
#define BSA_QUANTIZE_STATIC_SCRATCH_FLOATS (1 << 20)
int bsa_quantize_sage_static(const void* q, const void* k, const void* v, void* q8, void* k8, void* v8,
                             float* q_scale, float* k_scale, float* v_scale, int32_t B, int32_t H, int32_t Sq,
                             int32_t Sk, void* cuda_stream);

/*
 * Block mask -> q2k index.  mask [B,H,Nq,Nkv] uint8 (non-zero = attend).  Writes the attended KV block
 * ids of every row in ascending order to index [B,H,Nq,cap] (entries beyond the count are set to 0)
 * and the count to nums [B,H,Nq]; counts above cap are clamped.
 * The reference has no such function; the semantics are the inverse of the scatter in
 * tests/test_flash_fwd.py:156-170.
 */
int bsa_mask_to_q2k(const uint8_t* mask, int32_t* index, int32_t* nums, int32_t B, int32_t H,
                    int32_t Nq, int32_t Nkv, int32_t cap, void* cuda_stream);

/*
 * q2k -> dense k2q with set semantics: k2q_index [B,H,Nkv,Nq] ascending q ids, zero padded;
 * k2q_nums [B,H,Nkv].  Replaces convert_q2k_to_k2q_triton (utils/block_sparse_index.py:71-129).
 * q2k_nums may be NULL (count = block_sparse_num).
 */
int bsa_q2k_to_k2q(const int32_t* q2k_index, const int32_t* q2k_nums, int32_t block_sparse_num,
                   int32_t B, int32_t H, int32_t Nq, int32_t cap, int32_t Nkv, int32_t* k2q_index,
                   int32_t* k2q_nums, void* cuda_stream);

/*
 * Longest-first work order for skewed per-row counts: order[0..rows) = the row ids sorted by descending
 * clamp(q2k_nums[row], 0, cap), rows of equal count in ascending order (stable, deterministic).
 * scratch: bsa_lpt_order_scratch_ints(rows, cap) int32.  The reference has no counterpart: it balances
 * with the hardware work-stealing scheduler (csrc/utils/block_sparse_tile_scheduler.py:104-136).
 */
int bsa_lpt_order(const int32_t* q2k_nums, int32_t rows, int32_t cap, int32_t* order, int32_t* scratch,
                  void* cuda_stream);
int64_t bsa_lpt_order_scratch_ints(int32_t rows, int32_t cap);

/*
 * Top-k block selection, the step that produces the q2k index.  The reference has no kernel for it: its
 * benchmark builds the index with torch (tests/bench_cutedsl_performance.py:131-167: pooled scores ->
 * torch.topk(sorted=False) -> ascending sort -> int32) and its notes name the recipe (design/fp8/results.md:
 * 635-636: mean-pool, top-k, complete K-block index layout).
 *   bsa_block_mean:    x [B,H,S,D] bf16 with element strides (b,h,s; last stride 1) -> out [B,H,ceil(S/blk),D]
 *                      fp32, the mean of every blk consecutive tokens (a short tail averages what exists).
 *   bsa_pooled_scores: scores[bh,m,j] = scale * sum_d qm[bh,m,d] * km[bh,j,d], fp32, summed in ascending d.
 *   bsa_topk_q2k:      index[row, 0..k) = ids of the k largest scores of the row in ascending id order; among
 *                      equal scores the lower id wins, NaN ranks above +inf (torch.topk's convention);
 *                      index has row stride cap >= k, entries [k, cap) are left untouched.
 *                      Limits: Nkv <= BSA_TOPK_MAX_BLOCKS, k <= 4096.
 */
#define BSA_TOPK_MAX_BLOCKS 8192
int bsa_block_mean(const void* x, const int64_t* stride, int32_t B, int32_t H, int32_t S, int32_t D,
                   int32_t blk, float* out, void* cuda_stream);
int bsa_pooled_scores(const float* qm, const float* km, int32_t BH, int32_t Nq, int32_t Nkv, int32_t D,
                      float scale, float* scores, void* cuda_stream);
int bsa_topk_q2k(const float* scores, int64_t rows, int32_t Nkv, int32_t k, int32_t cap, int32_t* index,
                 void* cuda_stream);

/*
 * Bucketed k2q CSR for the backward pass.  offsets [B,H,G,Nkv+1] (running per (b,h) across the G
 * query groups of bucket_size_blocks q-blocks), indices [B,H,max(1,Nq*cap)] global q-block ids, every
 * CSR row in ascending q order (deterministic).  One edge per occurrence (q, position < count) whose id is
 * in [0,Nkv); negative counts act as 0, counts above cap are clamped.
 * Replaces the four kernels of csrc/bwd/bucketed_k2q_csr.py:114-238 (build_bucketed_k2q_csr_cutedsl :266-378).
 */
int bsa_build_k2q_csr(const int32_t* q2k_index, const int32_t* q2k_nums, int32_t block_sparse_num,
                      int32_t B, int32_t H, int32_t Nq, int32_t cap, int32_t Nkv,
                      int32_t bucket_size_blocks, int32_t* offsets, int32_t* indices,
                      void* cuda_stream);

/*
 * Backward pass, BF16, MHA, D = 128 (or 64 with blk = 128), blk = 128 or 64 tokens: dQ, dK, dV from dO, Q, K,
 * V, O, LSE.
 * Replaces the preprocess / main / postprocess callables of
 * csrc/bwd/sm100_blk128/bsa_bwd_sm100.py:2178-2385 (blk128) and of the blk64 driver
 * bsa_attn_interface.py:4022-4290 over csrc/bwd/sm100_blk64/bsa_bwd_sm100.py (preprocess
 * csrc/bwd/bsa_bwd_preprocess.py, postprocess csrc/bwd/bsa_bwd_postprocess.py).
 *   work_order_q / work_order_kv: NULL (natural order), or the order in which the persistent CTAs of the two
 *   main kernels walk their work items (CTA c takes entries c, 2G-1-c, 2G+c, ... of it, G = grid size); a
 *   longest-first order from bsa_lpt_order balances skewed per-row counts, as in the forward;
 *   block_sizes: NULL, or int32 valid-token counts of the KV blocks with element strides
 *   (bs_stride_b, bs_stride_h, 1); tokens beyond a block's count get no probability and zero dK / dV,
 *   exactly as the forward masks them (the reference's blk128 backward ignores block_sizes, its blk64
 *   backward honours them; here both do);
 *   csr_offsets / csr_indices as produced by bsa_build_k2q_csr with the same q2k metadata;
 *   workspace: bsa_bwd_workspace_bytes(...) bytes of device memory, contents unspecified on entry.
 * dQ is accumulated without atomics and in a fixed order, so repeated calls are bit-identical.
 */
typedef struct bsa_bwd_args {
  const void* dout;
  const void* q;
  const void* k;
  const void* v;
  const void* out;
  const float* lse;
  void* dq;
  void* dk;
  void* dv;
  const int32_t* q2k_index;
  const int32_t* q2k_nums;
  const int32_t* csr_offsets;
  const int32_t* csr_indices;
  const int32_t* block_sizes;
  const int32_t* work_order_q;  /* NULL, or a permutation of the B*H*Nq query tiles (dQ kernel) */
  const int32_t* work_order_kv; /* NULL, or a permutation of the B*H*Nkv KV blocks (dK/dV kernel) */
  void* workspace;
  int32_t* status;
  int64_t workspace_bytes;
  int64_t do_stride[3];
  int64_t q_stride[3];
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int64_t dq_stride[3];
  int64_t dk_stride[3];
  int64_t dv_stride[3];
  int64_t bs_stride_b;
  int64_t bs_stride_h;
  int32_t blk;
  int32_t B, H, Sq, Sk, D;
  int32_t cap;
  int32_t block_sparse_num;
  int32_t num_q_groups;
  int32_t bucket_size_blocks;
  float softmax_scale;
  int32_t stages; /* 0 = the whole backward; otherwise a mask of the passes to launch (bit 0 preprocess, bit 1 dQ,
                     bit 2 dK/dV), for timing one pass alone - the main passes read the preprocess results of an
                     earlier call from `workspace` */
} bsa_bwd_args;

int bsa_bwd(const bsa_bwd_args* args, void* cuda_stream);
int64_t bsa_bwd_workspace_bytes(int32_t B, int32_t H, int32_t Sq, int32_t Sk, int32_t D);

#ifdef __cplusplus
}
#endif
#endif /* BSA_B200_H_ */
