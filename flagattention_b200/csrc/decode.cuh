// Arguments of the decode-shaped split-KV partial kernel (see decode.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b200attn {

// Largest number of query rows per KV head (heads in the group x query positions) the
// register-resident kernel handles; above it the tensor-core path is used.
#ifndef B200ATTN_DECODE_MAX_ROWS
#define B200ATTN_DECODE_MAX_ROWS 2
#endif
constexpr int DECODE_MAX_ROWS = B200ATTN_DECODE_MAX_ROWS;
// Resident CTAs per SM the streaming kernel is compiled for (its minimum-blocks launch bound).
constexpr int decode_resident_ctas(int rows) { return rows <= 1 ? 3 : 2; }

struct DecodeArgs {
  const uint16_t* q;
  const uint16_t* k;
  const uint16_t* v;
  int64_t q_sb, q_sh, q_sm;  // element strides
  int64_t k_sb, k_sh, k_sn;
  int64_t v_sb, v_sh, v_sn;
  float* part_o;             // [B, Hq, num_splits, M, D] fp32, normalised within the split
  float* part_lse;           // [B, Hq, num_splits, M] natural-log normaliser of the split
  uint16_t* final_o;         // non-null (with num_splits == 1): write the result directly
  float* final_lse;
  int64_t o_sb, o_sh, o_sm;
  int B, Hq, Hkv, M, N, groups;
  int num_splits, keys_per_split;
  int causal;
  float qk_scale;            // sm_scale * log2(e)
  // Paged K/V (block_table != nullptr): k and v point at caches [num_blocks, Hkv, block, D]; key n of
  // sequence b lives in block block_table[b * bt_stride + (n >> block_shift)] at row n & (block - 1);
  // k_sb / v_sb are then the block strides and N is read per sequence from context_lens.
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* context_lens;
  int block_shift;
};

int launch_decode_partial(const DecodeArgs& a, int D, bool bf16, cudaStream_t stream);

}  // namespace b200attn
