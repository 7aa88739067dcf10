/*
 * C ABI of libb200attn: the sm_100a kernels behind flag_attn.flash_attention.
 *
 * Conventions
 *  - Every pointer in a params struct is a DEVICE pointer owned by the caller; the
 *    library allocates nothing, keeps no pointer after the call returns and only
 *    enqueues work on `stream` (a cudaStream_t passed as void*).
 *  - Tensors are addressed as [batch, head, row, feature] with four ELEMENT strides;
 *    the feature stride must be 1 and the other three multiples of 8 elements
 *    (16 bytes) with a 16-byte aligned base, because tiles are fetched by TMA.
 *  - Every function returns 0 on success and a negative B200ATTN_E* code otherwise;
 *    b200attn_last_error() then returns a thread-local message.
 *  - `status` (optional, may be NULL) is a device int32 the kernels set to a non-zero
 *    code when a bounded device-side wait gave up; it must be zero on entry.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_ABI_VERSION 3

enum {
  B200ATTN_OK = 0,
  B200ATTN_EINVAL = -1,       /* bad shape / stride / dtype / pointer          */
  B200ATTN_EUNSUPPORTED = -2, /* valid request the kernels do not implement    */
  B200ATTN_ECUDA = -3,        /* a CUDA runtime / driver call failed           */
  B200ATTN_ETIMEOUT = -4      /* device-side bounded wait expired (status word)*/
};

enum { B200ATTN_F16 = 0, B200ATTN_BF16 = 1, B200ATTN_F32 = 2 };

typedef struct {
  void* ptr;
  int64_t stride[4]; /* elements: batch, head, row, feature */
} b200attn_tensor;

/* Forward: replaces the launch of `_fwd_kernel` (flash.py:92-105, kernel flash.py:345-509).
 * o = softmax(q k^T * sm_scale [+causal mask]) [dropout] v ; lse = natural-log normaliser. */
typedef struct {
  b200attn_tensor q;   /* [B, Hq, M, D]  dtype                                   */
  b200attn_tensor k;   /* [B, Hkv, N, D] dtype                                   */
  b200attn_tensor v;   /* [B, Hkv, N, D] dtype                                   */
  b200attn_tensor o;   /* [B, Hq, M, D]  o_dtype (dtype, or F32)                 */
  float* lse;          /* [B, Hq, M] contiguous fp32                             */
  int32_t B, Hq, Hkv, M, N, D;
  int32_t dtype;       /* B200ATTN_F16 | B200ATTN_BF16                           */
  int32_t o_dtype;     /* dtype or B200ATTN_F32                                  */
  int32_t causal;      /* bottom-right aligned: key n visible iff n <= m + N - M */
  float sm_scale;
  float dropout_p;     /* 0 disables dropout                                     */
  uint64_t seed;       /* Philox key                                             */
  uint64_t offset;     /* Philox counter base                                    */
  int32_t* status;     /* optional device status word                            */
  /* Optional visibility band (band != 0), on top of `causal`: key n is visible to query m iff
   * dist_min <= m + (N - M) - n < dist_max. INT32_MIN / INT32_MAX leave that side open. Used for
   * the two regions of piecewise attention (piecewise.py:39-205: distance >= w takes the second
   * q/k pair) and usable as a sliding window. Rows with no visible key give o = 0, lse = -inf. */
  int32_t band, dist_min, dist_max;
  /* Optional (dropout_p > 0): b200attn_keep_mask_bytes() bytes that receive the keep decisions, one
   * bit per (query, key), for b200attn_bwd to reuse instead of re-evaluating Philox (the reference
   * recomputes them in both backward kernels, flash.py:660-664,846-850). NULL = not stored. */
  uint32_t* keep_mask;
} b200attn_fwd_params;

/* Size of the keep-decision cache: B * Hq * ceil(N / 32) * M words. */
size_t b200attn_keep_mask_bytes(int32_t B, int32_t Hq, int32_t M, int32_t N);

int b200attn_fwd(const b200attn_fwd_params* p, void* stream);

/* Total attention: replaces `_total_attention_kernel` (total.py:64-156, launched
 * flash.py:147-159). tot[b,h,n] = sum_m exp(s[m,n]*sm_scale - lse[m]) over visible m.
 * `workspace` is caller-allocated scratch of b200attn_total_workspace_bytes(B, Hq, M) bytes,
 * 16-byte aligned; its contents on entry do not matter. */
typedef struct {
  b200attn_tensor q;
  b200attn_tensor k;
  const float* lse;    /* [B, Hq, M] */
  float* tot;          /* [B, Hq, N] */
  void* workspace;
  int32_t B, Hq, Hkv, M, N, D;
  int32_t dtype;
  int32_t causal;
  float sm_scale;
  int32_t* status;
} b200attn_total_params;

size_t b200attn_total_workspace_bytes(int32_t B, int32_t Hq, int32_t M);
int b200attn_total_attention(const b200attn_total_params* p, void* stream);

/* Total attention for callers that cannot hand the library any scratch memory, e.g. a serving
 * process that gave its whole device-memory budget to its own pool at start-up, or a component
 * that is only passed input and output buffers and has no allocator to ask. No counterpart in the
 * reference. Same inputs, outputs and result as b200attn_total_attention; `workspace` is ignored.
 * The per-query statistics go to an array built into the library (B200ATTN_STATIC_STATS_MAX
 * entries, 4 MiB, held on every GPU that loads the library until the process exits), so the call
 * makes no device allocation of any kind.
 *  - Limit: B * Hq * roundup(M, 128) <= B200ATTN_STATIC_STATS_MAX, else B200ATTN_EUNSUPPORTED.
 *  - The first call on each device looks up the array's device address; make that first call
 *    outside any stream capture.
 *  - All calls share the one array per GPU and the array keeps what the last call wrote. Each call
 *    rewrites the part it reads before reading it, so nothing has to be cleared, but two calls
 *    whose kernels may run at the same time on one GPU (different streams) race on it. */
#define B200ATTN_STATIC_STATS_MAX 524288
int b200attn_total_attention_static(const b200attn_total_params* p, void* stream);

/* Backward: replaces `_bwd_preprocess`, `_bwd_kv_kernel`, `_bwd_q_kernel` and the GQA group
 * sum (flash.py:183-272, kernels flash.py:542-931).
 * `delta` [B,Hq,M] fp32 and `workspace` (b200attn_bwd_workspace_bytes() bytes, 16-byte aligned)
 * are caller-allocated scratch; their contents on entry do not matter. dK / dV are written
 * already summed over each KV head's query group (accumulated in fp32). */
typedef struct {
  b200attn_tensor q, k, v, o, d_o; /* o has o_dtype; d_o has dtype           */
  b200attn_tensor dq;              /* [B, Hq, M, D]  dtype                   */
  b200attn_tensor dk, dv;          /* [B, Hkv, N, D] dtype (group-summed)    */
  const float* lse;                /* [B, Hq, M]                             */
  float* delta;                    /* [B, Hq, M] scratch                     */
  void* workspace;                 /* b200attn_bwd_workspace_bytes() scratch  */
  int32_t B, Hq, Hkv, M, N, D;
  int32_t dtype, o_dtype;
  int32_t causal;
  float sm_scale;
  float dropout_p;
  uint64_t seed, offset;
  int32_t* status;
  int32_t band, dist_min, dist_max; /* visibility band as in b200attn_fwd_params */
  const uint32_t* keep_mask;        /* cache written by b200attn_fwd for the same call, or NULL */
  int32_t dv_accumulate;            /* != 0: dv already holds a gradient (16-bit); this call's dV is added to it in
                                       fp32 and the sum rounded once. Piecewise attention's two (q, k) pairs share
                                       one v (`piecewise.py:132-180` accumulates both regions into one dv) */
} b200attn_bwd_params;

size_t b200attn_bwd_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t M, int32_t N,
                                    int32_t D);
int b200attn_bwd(const b200attn_bwd_params* p, void* stream);

/* The same backward restricted to some of its stages, so a profiler or benchmark can time the
 * kernels one by one. PREP = delta + statistics preprocess, KV = the dK/dV kernel, Q = the dQ
 * kernel; KV and Q need the scratch PREP wrote. At D = 128 and 64 the KV stage is a fused pass that also
 * accumulates dQ in fp32 (in the workspace, by global reductions, so dQ is reproducible only up to
 * fp32 summation order) and the Q stage is the conversion of that accumulator; adding UNFUSED
 * selects the two separate kernels instead. The fused pass needs its accumulator
 * cleared: PREP clears it when it runs in the same call, otherwise the call clears it first unless
 * ACC_ZEROED says the caller has done so. No counterpart in the reference. */
enum {
  B200ATTN_BWD_STAGE_PREP = 1,
  B200ATTN_BWD_STAGE_KV = 2,
  B200ATTN_BWD_STAGE_Q = 4,
  B200ATTN_BWD_STAGE_ALL = 7,
  B200ATTN_BWD_STAGE_UNFUSED = 8,
  B200ATTN_BWD_STAGE_ACC_ZEROED = 16  /* the fp32 dQ accumulator (workspace bytes [B*Hq*roundup(M,128)*8,
                                         + B*Hq*M*D*4)) is already zero */
};
int b200attn_bwd_stages(const b200attn_bwd_params* p, void* stream, int32_t stages);

/* delta[b,h,m] = sum_d o*do in fp32: replaces `_bwd_preprocess` (flash.py:542-588). Also run
 * inside b200attn_bwd; exported for tests. */
int b200attn_bwd_delta(const b200attn_tensor* o, int32_t o_dtype, const b200attn_tensor* d_o,
                       int32_t do_dtype, float* delta, int32_t B, int32_t H, int32_t M, int32_t D,
                       void* stream);

/* Dropout keep-mask materialisation: replaces the test helper `recompute_mask_kernel`
 * (testing/dropout.py:19-39). mask[b,h,m,n] (uint8, contiguous) = 1 iff the element is kept. */
int b200attn_dropout_mask(uint8_t* mask, int32_t B, int32_t H, int32_t M, int32_t N, float dropout_p,
                          uint64_t seed, uint64_t offset, void* stream);

/* Split-KV forward + combine: replaces `_fwd_split_kv_kernel` / `_fwd_combine_kv_splits`
 * (split_kv.py:28-243, dispatched flash.py:106-144). part_o [B,Hq,S,M,D] fp32 and
 * part_lse [B,Hq,S,M] fp32 are caller-allocated scratch. */
typedef struct {
  b200attn_tensor q, k, v, o;
  float* lse;          /* [B, Hq, M] */
  float* part_o;       /* [B, Hq, S, M, D] fp32 scratch */
  float* part_lse;     /* [B, Hq, S, M] fp32 scratch    */
  int32_t B, Hq, Hkv, M, N, D;
  int32_t num_splits;  /* S >= 1 */
  int32_t dtype;
  int32_t causal;
  float sm_scale;
  int32_t* status;
} b200attn_splitkv_params;

int b200attn_fwd_splitkv(const b200attn_splitkv_params* p, void* stream);

/* Split count this library prefers for b200attn_fwd_splitkv on the current device (num_sms <= 0:
 * ask the device). Plays the role of `num_splits_herustic` (split_kv.py:245-278) for the public
 * `flash_attention_split_kv` (split_kv.py:282-347), but is tuned to this library's kernels: shapes
 * with at most 4 query rows per KV head (heads per group x M) run a register-resident streaming
 * kernel with several light CTAs per SM; grouped heads with up to 128 rows per KV head share one
 * tensor-core tile per KV head; everything else uses one tile pair per query head. The result of
 * the attention does not depend on the split count beyond fp32 rounding. Returns >= 1. */
int b200attn_splitkv_num_splits(int32_t B, int32_t Hq, int32_t Hkv, int32_t M, int32_t N, int32_t D,
                                int32_t num_sms);

/* Decode attention over a paged K/V cache: replaces `_paged_attn_kernel` + `_paged_attn_v2_reduce_kernel`
 * as launched by `paged.attention` (paged.py:20-170). One query row per sequence.
 *   q, o          [num_seqs, Hq, D] described as 4-D tensors [num_seqs, Hq, 1, D] (stride[2] unused)
 *   key_cache,
 *   value_cache   [num_blocks, Hkv, block_size, D]; key n of sequence s is row n % block_size of block
 *                 block_table[s * block_table_stride + n / block_size]
 *   context_lens  [num_seqs] int32, keys per sequence (<= max_context_len)
 *   lse           [num_seqs, Hq] fp32 out (log-normaliser; the reference does not return it)
 *   part_o/_lse   fp32 scratch [num_seqs, Hq, num_splits, D] / [num_seqs, Hq, num_splits], part_o
 *                 16-byte aligned; any num_splits >= 1 gives the same result up to fp32 rounding
 *                 (b200attn_splitkv_num_splits(num_seqs, Hq, Hkv, 1, max_context_len, D, 0) is the
 *                 tuned choice; the reference's own `num_splits` argument only tunes its kernels).
 * block_size must be a power of two (the reference accepts any size; its tests use 16, 128, 256),
 * and at least 8 when more than 2 query heads share a KV head. D in {16, 32, 64, 128} (the reference
 * also lists 256 and 512). Table entries beyond a sequence's last block are never read. */
typedef struct {
  b200attn_tensor q, key_cache, value_cache, o;
  const int32_t* block_table;
  int64_t block_table_stride;
  const int32_t* context_lens;
  float* lse;
  float* part_o;
  float* part_lse;
  int32_t num_seqs, Hq, Hkv, D, block_size, num_blocks, max_context_len, num_splits;
  int32_t dtype;
  float sm_scale;
  int32_t* status;
} b200attn_paged_params;

int b200attn_paged_attention(const b200attn_paged_params* p, void* stream);

/* Merge of two partial attention results over disjoint key sets, in place on the accumulator:
 * lse = log(exp(lse_acc) + exp(lse_part)), o_acc = o_acc*exp(lse_acc-lse) + o_part*exp(lse_part-lse).
 * Both sides are contiguous fp32 arrays [heads, rows_per_head, D] (o) and [heads, rows_per_head]
 * (lse); `rows` rows per head starting at acc_row0 / part_row0 take part. `first` != 0 treats
 * the accumulator rows as empty (they are overwritten). The algebra of `_fwd_combine_kv_splits`
 * (split_kv.py:199-231), used by the ring-KV sequence-parallel mode where the partials arrive one
 * ring step at a time. */
int b200attn_merge_partial(float* o_acc, float* lse_acc, const float* o_part, const float* lse_part,
                           int64_t heads, int32_t rows, int32_t D, int32_t acc_rows_per_head,
                           int32_t acc_row0, int32_t part_rows_per_head, int32_t part_row0,
                           int32_t first, void* stream);

/* The same merge for two complete partial results [B, H, M, D] (contiguous fp32, with fp32
 * log-normalisers [B, H, M]) whose sum is the final result: the merged rows are rounded straight into
 * the fp16/bf16 tensor `out` (own strides, 16-byte aligned rows) and `lse_a` receives the merged
 * log-normaliser. Used by piecewise attention's forward (the two regions of `piecewise.py:69-84`). */
int b200attn_merge_partial_store(const float* o_a, float* lse_a, const float* o_b, const float* lse_b,
                                 int32_t B, int32_t H, int32_t M, int32_t D, const b200attn_tensor* out,
                                 int32_t out_dtype, void* stream);

/* Diagnostics. */
int b200attn_abi_version(void);
const char* b200attn_last_error(void);

/* One 128xN tcgen05 tile product with caller-chosen descriptor fields; used by the GPU
 * tests to pin the shared-memory / TMEM operand layouts the attention kernels rely on.
 * No counterpart in the reference. */
typedef struct {
  const void* a;       /* [128, a_cols] row-major 16-bit          */
  const void* b;       /* [b_rows, b_cols] row-major 16-bit       */
  float* d;            /* [128, n] fp32 out                       */
  int32_t a_cols, b_rows, b_cols;
  int32_t box_cols;    /* TMA box width in elements (<= 64)       */
  int32_t swizzle;     /* 0 none, 1 32B, 2 64B, 3 128B (TMA enum) */
  int32_t bf16;
  int32_t a_in_tmem;   /* 0: A from smem; 1: A stored to TMEM by threads; 2: smem -> TMEM by tcgen05.cp */
  int32_t n;           /* MMA N                                   */
  int32_t k_steps;     /* number of K=16 MMAs                     */
  uint32_t idesc;
  uint64_t a_desc_hi, b_desc_hi;   /* descriptor bits above the address   */
  int32_t a_step_bytes, b_step_bytes; /* start-address advance per K step */
  int32_t a_chunk_steps, b_chunk_steps; /* K steps per TMA chunk (0 = all in one) */
  int32_t a_chunk_bytes, b_chunk_bytes; /* byte jump between chunks                */
  int32_t* status;
} b200attn_selftest_params;

int b200attn_umma_selftest(const b200attn_selftest_params* p, void* stream);

/* Exercises, harmlessly, what every kernel does when one of its bounded device-side waits runs out:
 * one small CTA waits at most `limit_us` (1..1000) microseconds on a barrier that nothing arrives at,
 * records `code` (1..4, the kernels' status codes) in `*status`, releases its other warps through the
 * abort flag, frees its TMEM and returns; the context stays usable. `out` (3 device int64): [0] = 1 if
 * the wait gave up, [1] = warps released by the abort flag (3 expected), [2] = nanoseconds waited.
 * No counterpart in the reference. */
int b200attn_wait_timeout_selftest(int32_t limit_us, int32_t code, int32_t* status, long long* out,
                                   void* stream);

/* Host-only check (no GPU needed) of the prepared divisions with which the kernels turn a work-item
 * number into (batch, head) pair and row block: `pairs` pairs x `n_z` row blocks, visited in chunks
 * of `chunk` pairs. Returns the number of item numbers that decode differently from plain integer
 * division (0 = correct), or a negative code for bad arguments. No counterpart in the reference. */
int b200attn_work_order_selftest(int32_t pairs, int32_t n_z, int32_t chunk);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
