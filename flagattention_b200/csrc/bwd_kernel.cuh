// Backward / total-attention kernel family for sm_100a.
//
// One kernel template, three modes. In every mode a CTA owns 128 "row" indices whose tiles stay
// resident in shared memory, and streams 64 "column" indices per step through a TMA ring:
//
//   MODE_KV    rows = keys n of one KV head, columns = queries m of every query head of its group.
//              T1 = K Q^T, T2 = V dO^T (so probabilities come out transposed, key on the TMEM
//              lane), dV += P^T dO, dK += dS^T Q. The group sum of dK/dV happens in the fp32
//              accumulators. Replaces `_bwd_kv_kernel` (flash.py:591-765) + the sum at :270-271.
//   MODE_Q     rows = queries m of one query head, columns = keys n.
//              T1 = Q K^T, T2 = dO V^T, dQ += dS K. Replaces `_bwd_q_kernel` (flash.py:768-931).
//   MODE_TOTAL rows = keys n of one query head's KV head, columns = queries m.
//              T1 = K Q^T, tot[n] = sum_m P. Replaces `_total_attention_kernel` (total.py:64-156).
//
// P is recomputed as exp2(T1*qk_scale - lse*log2e) and dS = P * (dP - delta), with dropout applied
// as in the reference (dV uses the masked P and is scaled by 1/(1-p) at the end; dP is masked and
// scaled by 1/(1-p) before delta is subtracted).
//
// Roles: warps 0-3 and 4-7 are two softmax groups that alternate steps (thread r <-> row r), warp 8
// issues tcgen05.mma, warp 9 drives TMA. TMEM: accumulators (D columns each) followed by two
// (T1, T2) buffers of 64+64 fp32 columns; P / dS overwrite T1 as packed 16-bit pairs and are
// consumed from TMEM as the A operand of the accumulating MMAs.
//
// FUSED (MODE_KV, D = 128 and 64): the same pass also produces dQ, so P and dS are computed once for
// the whole backward. The softmax groups leave dS^T a second time in shared memory ([128 keys x 64
// queries], 128-byte swizzled rows); the MMA warp forms dQ^T = K^T dS^T (A = the resident K tile read
// MN-major, 128 x 64 fp32) in the step's dead T2 columns (D = 128) or in columns of its own (D = 64),
// ahead of the step's accumulating products
// so that the read-back overlaps them; four extra warps read it back, transpose it through two
// 16 KB staging tiles ([32 queries][128 features] fp32, the layout of the accumulator rows) and add
// it to an fp32 dQ accumulator in global memory with cp.reduce.async.bulk (.add.f32), since every
// key block contributes to every query row. A conversion kernel scales and rounds the accumulator
// afterwards. The reductions (32 KB per step and SM) run at the rate the L2 accepts them, about
// 13 bytes per clock and SM, which is what bounds this pass.
//
// Per-query statistics come from a padded scratch array holding, per pair of queries, the float4
// (-lse[m]*log2e, -lse[m+1]*log2e, -delta[m], -delta[m+1]); it is padded to a multiple of 128
// queries with (-inf, 0) so that padded and key-less queries contribute exactly zero. The pair
// layout feeds the packed f32x2 arithmetic of the recompute loop directly.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "fwd_kernel.cuh"
#include "ptx.cuh"

namespace b200attn {

enum BwdMode : int { MODE_KV = 0, MODE_Q = 1, MODE_TOTAL = 2 };

struct BwdArgs {
  void* out1;  // MODE_KV: dK, MODE_Q: dQ
  void* out2;  // MODE_KV: dV
  int64_t out1_sb, out1_sh, out1_sr;
  int64_t out2_sb, out2_sh, out2_sr;
  const float2* stats;  // [B, Hq, Mpad/2] float4 pairs, see above
  float* tot;           // MODE_TOTAL: [B, Hq, N]
  int B, Hq, Hkv, M, N, Mpad, groups, causal;  // causal: some band limit below is finite
  int d_min, d_max;  // visibility band: query m sees key n iff d_min <= m + (N - M) - n < d_max
  int n_zblocks, grid_chunk;  // grid order, see decode_block()
  float sm_scale, qk_scale;
  DropoutCtx drop;
  int32_t* status;
  float* dq_acc;        // FUSED: [B, Hq, M, D] fp32, zero before the launch
  int out_tma;          // the 16-bit results leave through shared memory and TMA stores (tmO1, tmO2)
  int out2_accumulate;  // MODE_KV: out2 (dV) already holds a 16-bit gradient that this pass adds to
};

template <int D, int MODE, bool FUSED = false>
struct BwdSmem {
  static constexpr int STAGES = (FUSED && D == 128) ? 3 : 4;
  static constexpr int N_A = MODE == MODE_TOTAL ? 1 : 2;       // resident tiles
  static constexpr int N_B = MODE == MODE_TOTAL ? 1 : 2;       // streamed tiles per stage
  static constexpr int A_BYTES = N_A * TileCfg<D>::TILE_BYTES; // 128 x D each
  static constexpr int B_TILE_BYTES = 64 * D * 2;
  static constexpr int STATS_BYTES = MODE == MODE_Q ? 0 : 512; // 64 x float2
  static constexpr int STAGE_BYTES = N_B * B_TILE_BYTES + 1024; // tiles + stats slot (keeps 1 KB alignment)
  static constexpr int DS_TILE_BYTES = 128 * 128;               // FUSED: dS^T, 128 keys x 64 queries
  static constexpr int DS_OFFSET = A_BYTES + STAGES * STAGE_BYTES;
  static constexpr int DQ_STAGE_BYTES = 32 * D * 4;             // FUSED: 32 queries x D fp32 of dQ on its way out
  static constexpr int DQ_STAGE_OFFSET = DS_OFFSET + (FUSED ? DS_TILE_BYTES : 0);
  static constexpr int BAR_OFFSET = DQ_STAGE_OFFSET + (FUSED ? 2 * DQ_STAGE_BYTES : 0);
  static constexpr int TOTAL = BAR_OFFSET + 512 + 1024;
  static constexpr int THREADS = FUSED ? 448 : 320;
};

template <int D, bool BF16, bool DROPOUT, int MODE, bool FUSED = false>
__global__ void __launch_bounds__((BwdSmem<D, MODE, FUSED>::THREADS), 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmA2,
           const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
           const __grid_constant__ CUtensorMap tmO1, const __grid_constant__ CUtensorMap tmO2,
           const BwdArgs args) {
  using Cfg = TileCfg<D>;
  using Sm = BwdSmem<D, MODE, FUSED>;
  static_assert(!FUSED || (MODE == MODE_KV && (D == 128 || D == 64)),
                "the fused dQ pass exists for MODE_KV, D = 128 and 64");
  constexpr int STAGES = Sm::STAGES;
  constexpr int STEP = 64;                                  // columns per step
  constexpr int CHUNK_BYTES_B = STEP * Cfg::ROW_BYTES;      // one [64 x CHUNK] box
  constexpr uint64_t MN_DESC_B = make_smem_desc_hi(CHUNK_BYTES_B, 8 * Cfg::ROW_BYTES, Cfg::UMMA_SWZ);
  constexpr int N_ACC = MODE == MODE_KV ? 2 : (MODE == MODE_Q ? 1 : 0);
  constexpr uint32_t BUF_BASE = N_ACC * D;                  // TMEM column of buffer 0
  // When TMEM has room, the resident tiles are copied into it once (tcgen05.cp) and the T products
  // read their A operand from there: with 64-column steps those products are otherwise limited by
  // shared-memory bandwidth (both operands streamed from shared memory for every step).
  constexpr uint32_t A_BASE = BUF_BASE + 256;               // TMEM column of the resident copies
  constexpr bool A_IN_TMEM = A_BASE + Sm::N_A * (D / 2) <= 512;
  // FUSED: where dQ^T (64 fp32 columns) lives. D = 128 has no free columns, so it takes the step's
  // T2 columns once dP^T has been consumed; D = 64 has 64 columns left after the resident copies.
  constexpr bool DQ_ALIASED = D == 128;
  constexpr uint32_t DQ_COL_FIXED = A_BASE + Sm::N_A * (D / 2);
  static_assert(!FUSED || DQ_ALIASED || DQ_COL_FIXED + 64 <= 512, "no TMEM columns for dQ^T");
  auto dq_col = [](int buf) -> uint32_t { return DQ_ALIASED ? BUF_BASE + buf * 128 + 64 : DQ_COL_FIXED; };
  // (single fixed buffer: one barrier pair, phase = step parity; aliased: one pair per T buffer)
  auto dq_slot = [](int i) -> int { return DQ_ALIASED ? (i & 1) : 0; };
  auto dq_phase = [](int i) -> uint32_t { return DQ_ALIASED ? ((i >> 1) & 1) : (i & 1); };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + Sm::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Sm::BAR_OFFSET);
  uint64_t* a_full = bars;                 // [1]
  uint64_t* b_full = bars + 1;             // [STAGES]
  uint64_t* b_empty = b_full + STAGES;     // [STAGES]
  uint64_t* t_full = b_empty + STAGES;     // [2]
  uint64_t* p_ready = t_full + 2;          // [2]
  uint64_t* acc_full = p_ready + 2;        // [1]
  uint64_t* dq_ready = acc_full + 1;       // [2] FUSED: dQ^T of the step is complete in TMEM
  uint64_t* dq_drained = dq_ready + 2;     // [2] FUSED: ... and has been read back
  uint64_t* epi_sync = dq_drained + 2;     // [1] the eight softmax warps meet here before the output stores
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_sync + 1);
  uint8_t* sDS = smem + Sm::DS_OFFSET;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int P_SEQ = args.N - args.M;

  // Row block, the heads it loops over and its column range [col_lo, col_hi) in steps of 64.
  int r0, h_first, n_heads, hk, col_lo, col_hi;
  const int grid_heads = MODE == MODE_KV ? args.Hkv : args.Hq;
  const BlockCoord bc = decode_block(blockIdx.x, args.B * grid_heads, args.n_zblocks, args.grid_chunk);
  const int b = bc.bh / grid_heads;
  const int grid_h = bc.bh % grid_heads;
  if constexpr (MODE == MODE_Q) {
    r0 = (args.n_zblocks - 1 - bc.z) * 128;  // longest (causal) blocks first
    h_first = grid_h;
    n_heads = 1;
    hk = h_first / args.groups;
    col_lo = 0;
    col_hi = (args.causal && args.d_min > -BAND_INF) ? min(args.N, max(0, P_SEQ + r0 + 128 - args.d_min)) : args.N;
    if (args.causal && args.d_max < BAND_INF) col_lo = min(col_hi, (max(0, r0 + P_SEQ - args.d_max + 1) / STEP) * STEP);
  } else {
    r0 = bc.z * 128;                          // small n0 = most visible queries = longest first
    if constexpr (MODE == MODE_KV) {
      hk = grid_h;
      h_first = hk * args.groups;
      n_heads = args.groups;
    } else {
      h_first = grid_h;
      n_heads = 1;
      hk = h_first / args.groups;
    }
    col_lo = (args.causal && args.d_min > -BAND_INF) ? (max(0, r0 - P_SEQ + args.d_min) / STEP) * STEP : 0;
    col_hi = (args.causal && args.d_max < BAND_INF) ? min(args.M, max(0, r0 + 127 - P_SEQ + args.d_max)) : args.M;
  }
  const int steps_per_head = col_hi > col_lo ? cdiv(col_hi - col_lo, STEP) : 0;
  const int T = steps_per_head * n_heads;

  if (threadIdx.x == 0) {
    mbar_init(a_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&p_ready[i], 256);
      mbar_init(&dq_ready[i], 1);
      mbar_init(&dq_drained[i], 128);
    }
    mbar_init(acc_full, 1);
    mbar_init(epi_sync, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto fail = [&](int32_t code) {
    report_status(args.status, code);
    *abort_flag = 1;
  };
  auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
    return bounded_wait(bar, parity, abort_flag, args.status, WAIT_LIMIT_NS);
  };

  if (warp == 9) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && T > 0) {
      tma_prefetch_desc(&tmA1);
      tma_prefetch_desc(&tmB1);
      if constexpr (MODE != MODE_TOTAL) {
        tma_prefetch_desc(&tmA2);
        tma_prefetch_desc(&tmB2);
      }
      const int a_head = MODE == MODE_Q ? h_first : hk;
      mbar_expect_tx(a_full, Sm::A_BYTES);
      for (int c = 0; c < Cfg::NCHUNK; ++c) {
        tma_load_4d(sA + c * Cfg::CHUNK_BYTES, &tmA1, a_full, c * Cfg::CHUNK, r0, a_head, b);
        if constexpr (MODE != MODE_TOTAL)
          tma_load_4d(sA + Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmA2, a_full, c * Cfg::CHUNK, r0,
                      a_head, b);
      }
      for (int i = 0; i < T; ++i) {
        const int st = i % STAGES;
        const int hh = i / steps_per_head;
        const int col = col_lo + (i - hh * steps_per_head) * STEP;
        const int b_head = MODE == MODE_Q ? hk : h_first + hh;
        if (!wait(&b_empty[st], ((i / STAGES) & 1) ^ 1)) { fail(ST_WAIT_EMPTY); break; }
        uint8_t* stage = sB + st * Sm::STAGE_BYTES;
        mbar_expect_tx(&b_full[st], Sm::N_B * Sm::B_TILE_BYTES + Sm::STATS_BYTES);
        for (int c = 0; c < Cfg::NCHUNK; ++c) {
          tma_load_4d(stage + c * CHUNK_BYTES_B, &tmB1, &b_full[st], c * Cfg::CHUNK, col, b_head, b);
          if constexpr (MODE != MODE_TOTAL)
            tma_load_4d(stage + Sm::B_TILE_BYTES + c * CHUNK_BYTES_B, &tmB2, &b_full[st],
                        c * Cfg::CHUNK, col, b_head, b);
        }
        if constexpr (MODE != MODE_Q) {
          const float2* src = args.stats + (static_cast<int64_t>(b) * args.Hq + b_head) * args.Mpad + col;
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
              ::"r"(smem_u32(stage + Sm::N_B * Sm::B_TILE_BYTES)),
              "l"(reinterpret_cast<uint64_t>(src)), "r"(512), "r"(smem_u32(&b_full[st]))
              : "memory");
        }
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------------------------------------------- MMA issuer
    // The whole warp runs this loop with warp-uniform values; one elected lane issues each
    // tcgen05 instruction (see mma_ss_w).
    if (T > 0) {
      constexpr uint32_t IDESC_T = make_idesc(BF16, 128, STEP, false, false);
      constexpr uint32_t IDESC_ACC = make_idesc(BF16, 128, D, false, true);
      const uint32_t a_addr = smem_u32(sA);
      const uint32_t b_addr = smem_u32(sB);
      // T1 = A1 B1^T, T2 = A2 B2^T into buffer `buf` from ring stage `st`.
      auto a_offset = [](int which, int s) -> uint32_t {
        return which * Cfg::TILE_BYTES + (s / Cfg::STEPS_PER_CHUNK) * Cfg::CHUNK_BYTES +
               (s % Cfg::STEPS_PER_CHUNK) * 32;
      };
      // Resident tiles -> TMEM, one K=16 slice (8 columns) per copy.
      auto stage_resident = [&]() {
        const uint64_t da = smem_desc(Cfg::KMAJOR_DESC, a_addr);
#pragma unroll
        for (int which = 0; which < Sm::N_A; ++which) {
#pragma unroll
          for (int s = 0; s < D / 16; ++s)
            tmem_cp_128x256b_w(tmem_base + A_BASE + which * (D / 2) + s * 8, da + (a_offset(which, s) >> 4));
        }
      };
      auto issue_t = [&](int buf, int st) {
        const uint32_t t1 = tmem_base + BUF_BASE + buf * 128;
        const uint64_t da = smem_desc(Cfg::KMAJOR_DESC, a_addr);
        const uint64_t db = smem_desc(Cfg::KMAJOR_DESC, b_addr + st * Sm::STAGE_BYTES);
#pragma unroll
        for (int which = 0; which < Sm::N_A; ++which) {
#pragma unroll
          for (int s = 0; s < D / 16; ++s) {
            const uint32_t b_off = which * Sm::B_TILE_BYTES + (s / Cfg::STEPS_PER_CHUNK) * CHUNK_BYTES_B +
                                   (s % Cfg::STEPS_PER_CHUNK) * 32;
            // offsets are multiples of 16 bytes and stay inside shared memory, so they add into
            // the 14-bit address field without carrying out of it
            if constexpr (A_IN_TMEM) {
              mma_ts_w(t1 + which * 64, tmem_base + A_BASE + which * (D / 2) + s * 8, db + (b_off >> 4),
                       IDESC_T, s > 0 ? 1u : 0u);
            } else {
              mma_ss_w(t1 + which * 64, da + (a_offset(which, s) >> 4), db + (b_off >> 4), IDESC_T,
                       s > 0 ? 1u : 0u);
            }
          }
        }
      };
      // acc[which] += (P or dS from TMEM) x streamed tile `tile` of stage `st`, read MN-major.
      auto issue_acc = [&](int acc, int buf, int src, int st, int tile, bool accumulate) {
        const uint32_t d = tmem_base + acc * D;
        // Softmax group g leaves its 32 columns' P (8+8 packed columns) at T1[32g, 32g+16) and
        // its dS at T1[32g+16, 32g+32): K-step s covers columns 16s..16s+15 of the step.
        const uint32_t a = tmem_base + BUF_BASE + buf * 128 + src * 16;
        const uint64_t db = smem_desc(MN_DESC_B, b_addr + st * Sm::STAGE_BYTES + tile * Sm::B_TILE_BYTES);
#pragma unroll
        for (int s = 0; s < STEP / 16; ++s)
          mma_ts_w(d, a + (s >> 1) * 32 + (s & 1) * 8, db + ((s * 16 * Cfg::ROW_BYTES) >> 4), IDESC_ACC,
                   (accumulate || s > 0) ? 1u : 0u);
      };
      // FUSED: dQ^T (feature rows x 64 queries) = K^T dS^T. The product always has M = 128: at
      // D = 64 the MN-major descriptor runs on from the K tile into the V tile behind it, so lanes
      // 64..127 receive V^T dS^T, which nobody reads.
      auto issue_dq = [&](int buf) {
        constexpr uint32_t IDESC_DQ = make_idesc(BF16, 128, STEP, true, true);
        constexpr uint64_t DS_DESC = make_smem_desc_hi(Sm::DS_TILE_BYTES, 1024, SWZ_128B);
        const uint64_t da = smem_desc(Cfg::MNMAJOR_DESC, a_addr);  // K, rows = contraction index
        const uint64_t db = smem_desc(DS_DESC, smem_u32(sDS));
#pragma unroll
        for (int s = 0; s < 128 / 16; ++s)
          mma_ss_w(tmem_base + dq_col(buf), da + ((s * 16 * Cfg::ROW_BYTES) >> 4),
                   db + ((s * 16 * 128) >> 4), IDESC_DQ, s > 0 ? 1u : 0u);
      };
      bool ok = true;
      if (!wait(a_full, 0)) { fail(ST_WAIT_TMA); ok = false; }
      if (ok && !wait(&b_full[0], 0)) { fail(ST_WAIT_TMA); ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        if constexpr (A_IN_TMEM) stage_resident();
        issue_t(0, 0);
        tc_commit_w(&t_full[0]);
      }
      for (int i = 0; i < T && ok; ++i) {
        const int buf = i & 1;
        const int st = i % STAGES;
        if (i + 1 < T) {
          const int st_next = (i + 1) % STAGES;
          const bool w = wait(&b_full[st_next], ((i + 1) / STAGES) & 1);
          if (!__all_sync(0xffffffffu, w)) { fail(ST_WAIT_TMA); ok = false; break; }
          if constexpr (FUSED && DQ_ALIASED) {
            // the T2 columns of the other buffer still hold dQ^T of step i - 1 until it is read back
            if (i >= 1) {
              const bool w2 = wait(&dq_drained[dq_slot(i - 1)], dq_phase(i - 1));
              if (!__all_sync(0xffffffffu, w2)) { fail(ST_WAIT_SOFTMAX); ok = false; break; }
            }
          }
          tc_fence_after();
          issue_t(buf ^ 1, st_next);
          tc_commit_w(&t_full[buf ^ 1]);
        }
        {
          const bool w = wait(&p_ready[buf], (i >> 1) & 1);
          if (!__all_sync(0xffffffffu, w)) { fail(ST_WAIT_SOFTMAX); ok = false; break; }
        }
        tc_fence_after();
        if constexpr (MODE == MODE_KV) {
          if constexpr (FUSED) {
            if constexpr (!DQ_ALIASED) {
              // one fixed dQ^T buffer: the previous step's must have been read back
              if (i >= 1) {
                const bool w2 = wait(&dq_drained[0], dq_phase(i - 1));
                if (!__all_sync(0xffffffffu, w2)) { fail(ST_WAIT_SOFTMAX); ok = false; break; }
                tc_fence_after();
              }
            }
            // first, so that its read-back overlaps the two accumulating products and (aliased)
            // the T2 columns are free again when the next T products are issued
            issue_dq(buf);
            tc_commit_w(&dq_ready[dq_slot(i)]);
          }
          issue_acc(1, buf, 0, st, 1, i > 0);  // dV += P^T  dO
          issue_acc(0, buf, 1, st, 0, i > 0);  // dK += dS^T Q
        } else if constexpr (MODE == MODE_Q) {
          issue_acc(0, buf, 1, st, 0, i > 0);  // dQ += dS K
        }
        tc_commit_w(&b_empty[st]);
      }
      if (ok) tc_commit_w(acc_full);
    }
    __syncwarp();
  } else if (warp >= 10) {
    // ------------------------------------------------- FUSED: dQ^T read-back and global reduction
    if constexpr (FUSED) {
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const int d = (warp & 3) * 32 + lane;  // feature index = TMEM lane
      for (int i = 0; i < T; ++i) {
        const int buf = i & 1;
        const int hh = i / steps_per_head;
        const int col = col_lo + (i - hh * steps_per_head) * STEP;
        {
          // The four warps decide together whether to go on: they meet at named barriers below, so
          // one of them leaving alone would strand the others there. Each warp's own wait is bounded,
          // hence all four reach this reduction barrier.
          const bool w = wait(&dq_ready[dq_slot(i)], dq_phase(i));
          uint32_t all_ok;
          asm volatile(
              "{\n\t"
              ".reg .pred p, q;\n\t"
              "setp.ne.b32 p, %1, 0;\n\t"
              "bar.red.and.pred q, 2, 128, p;\n\t"
              "selp.b32 %0, 1, 0, q;\n\t"
              "}\n"
              : "=r"(all_ok) : "r"(static_cast<uint32_t>(w)) : "memory");
          if (!all_ok) { if (!w) fail(ST_WAIT_MMA); break; }
        }
        tc_fence_after();
        uint32_t v[STEP];
        tmem_ld32(tmem_base + lane_base + dq_col(buf), v);
        tmem_ld32(tmem_base + lane_base + dq_col(buf) + 32, v + 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&dq_drained[dq_slot(i)]);
        // Out through shared memory, 32 queries at a time: the tile is laid out like the
        // accumulator rows ([query][feature], contiguous in global memory) and one bulk
        // reduction adds it to the fp32 accumulator.
        float* dst = args.dq_acc + ((static_cast<int64_t>(b) * args.Hq + h_first + hh) * args.M + col) * D;
        const int n_valid = min(STEP, args.M - col);
        float* stage0 = reinterpret_cast<float*>(smem + Sm::DQ_STAGE_OFFSET);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int rows_out = min(32, n_valid - half * 32);
          // two staging tiles: this one was last read by the reduction issued two halves ago
          if (threadIdx.x == 320) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          asm volatile("bar.sync 2, 128;" ::: "memory");
          float* stage = stage0 + half * (Sm::DQ_STAGE_BYTES / 4);
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (d < D) stage[c * D + d] = __uint_as_float(v[half * 32 + c]);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 2, 128;" ::: "memory");
          if (threadIdx.x == 320 && rows_out > 0) {
            asm volatile(
                "cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                ::"l"(dst + half * 32 * D), "r"(smem_u32(stage)), "r"(rows_out * D * 4)
                : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
      // the staging tile must outlive the reductions that read it
      if (threadIdx.x == 320) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else {
    // --------------------------------------------------------- softmax groups
    const int wg = warp >> 2;
    const int row_local = (warp & 3) * 32 + lane;
    const int row = r0 + row_local;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float qk_scale = args.qk_scale;
    float row_nlse = -INFINITY, row_ndelta = 0.f;   // MODE_Q: this row's -lse*log2e and -delta
    if constexpr (MODE == MODE_Q) {
      if (row < args.Mpad) {
        const float* st = reinterpret_cast<const float*>(args.stats) +
                          ((static_cast<int64_t>(b) * args.Hq + h_first) * args.Mpad + (row & ~1)) * 2;
        row_nlse = st[row & 1];
        row_ndelta = st[2 + (row & 1)];
      }
    }
    const uint64_t scale2 = f2_pack(qk_scale, qk_scale);
    float tot_sum = 0.f;
    bool ok = true;
    // The band limits of this thread with "key n < N" folded in, so that masking keys past the end
    // costs no instruction per score: with keys on the rows a thread past the end sees nothing; with
    // keys on the columns n < N is the distance bound d = m + P_SEQ - n > m - M.
    const int my_d_min = MODE == MODE_Q ? max(args.d_min, row - args.M + 1) : args.d_min;
    const int my_d_max = (MODE != MODE_Q && row >= args.N) ? -BAND_INF - 2 : args.d_max;

    // Both groups work on every step: group `wg` owns columns [32*wg, 32*wg + 32) of the step, which
    // halves the latency between the T products and the accumulating products of a step.
    constexpr int HALF = STEP / 2;
    for (int i = 0; i < T; ++i) {
      const int st = i % STAGES;
      const int buf = i & 1;
      const int hh = i / steps_per_head;
      const int col0 = col_lo + (i - hh * steps_per_head) * STEP + wg * HALF;  // first column of this group
      const int h = h_first + hh;
      const uint32_t t1_addr = tmem_base + lane_base + BUF_BASE + buf * 128;
      // Dropout decisions for this thread's 32 (row, column) pairs of the step, generated before the
      // T products are awaited so the integer work overlaps the tensor core.
      uint32_t keep_bits = 0xffffffffu;
      if constexpr (DROPOUT) {
        const uint64_t head_base = args.drop.offset +
                                   (static_cast<uint64_t>(b) * args.Hq + h) * args.M * static_cast<uint64_t>(args.N);
        if (args.drop.keep_mask != nullptr) {
          // decisions cached by the forward (see DropoutCtx::keep_mask)
          const uint32_t* mk = args.drop.keep_mask + (static_cast<int64_t>(b) * args.Hq + h) * args.drop.mask_words * args.M;
          if constexpr (MODE == MODE_Q) {
            keep_bits = row < args.M ? mk[static_cast<int64_t>(col0 >> 5) * args.M + row] : 0u;
          } else {
            // the warp's 32 key rows share one word index; lane c fetches query col0 + c's word (bit l =
            // key l of the warp), and a 32 x 32 bit transpose across the warp (five butterfly steps)
            // leaves in lane l the word whose bit c is the decision for (key l, query col0 + c)
            const int wi = (r0 + (warp & 3) * 32) >> 5;
            keep_bits = (col0 + lane < args.M && wi < args.drop.mask_words)
                            ? mk[static_cast<int64_t>(wi) * args.M + col0 + lane] : 0u;
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) {
              const uint32_t m = s == 16 ? 0x0000ffffu : s == 8 ? 0x00ff00ffu : s == 4 ? 0x0f0f0f0fu
                                 : s == 2 ? 0x33333333u : 0x55555555u;
              const uint32_t y = __shfl_xor_sync(0xffffffffu, keep_bits, s);
              keep_bits = (lane & s) ? ((keep_bits & ~m) | ((y >> s) & m)) : ((keep_bits & m) | ((y << s) & ~m));
            }
          }
        } else if constexpr (MODE == MODE_Q) {
          keep_bits = dropout_keep_word(args.drop, head_base + static_cast<uint64_t>(row) * args.N + col0);
        } else {
          keep_bits = dropout_keep_word_strided(args.drop, head_base + static_cast<uint64_t>(col0) * args.N + row,
                                                static_cast<uint64_t>(args.N));
        }
      }
      {
        const bool w = wait(&t_full[buf], (i >> 1) & 1);
        if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_MMA); ok = false; break; }
      }
      tc_fence_after();
      uint32_t t1[HALF];
      uint32_t t2[MODE == MODE_TOTAL ? 1 : HALF];
      tmem_ld32(t1_addr + wg * HALF, t1);
      if constexpr (MODE != MODE_TOTAL) tmem_ld32(t1_addr + 64 + wg * HALF, t2);
      tmem_wait_ld();

      // Does this step cross the causal boundary for some row of the block?
      bool diag = false;
      if (args.causal) {
        // d = m + P_SEQ - n ranges over [d_lo_blk, d_hi_blk] on this group's 128 x 32 block
        int d_lo_blk, d_hi_blk;
        if constexpr (MODE == MODE_Q) {
          d_lo_blk = r0 + P_SEQ - (col0 + HALF - 1);
          d_hi_blk = r0 + 127 + P_SEQ - col0;
        } else {
          d_lo_blk = col0 + P_SEQ - (r0 + 127);
          d_hi_blk = col0 + HALF - 1 + P_SEQ - r0;
        }
        diag = d_lo_blk < args.d_min || d_hi_blk >= args.d_max;
      }
      // Keys past the end of the sequence: their K and V rows are zero-filled by TMA, so the recomputed
      // score is 0 and P = exp(-lse), which is not zero and overflows the 16-bit P (and with it dS, and
      // through 0 x inf the whole dQ row) when a query's log-normaliser is very negative. Mask them like
      // hidden entries.
      if constexpr (MODE == MODE_Q) {
        diag = diag || col0 + HALF > args.N;
      } else {
        diag = diag || r0 + 128 > args.N;
      }
      const float4* stats4 = reinterpret_cast<const float4*>(sB + st * Sm::STAGE_BYTES + Sm::N_B * Sm::B_TILE_BYTES) +
                             wg * (HALF / 2);
      // The loop exists twice, with and without the per-score visibility test, chosen once per step:
      // left as a test of `diag` inside the loop it is compiled into predicated instructions that every
      // step issues, masked or not (two more operations per pair there cost the whole pass 8 %).
      auto recompute = [&](auto diag_tag) {
        constexpr bool DIAG = decltype(diag_tag)::value;
#pragma unroll
        for (int c = 0; c < HALF; c += 2) {
          uint64_t nlse2, ndel2;
          if constexpr (MODE == MODE_Q) {
            nlse2 = f2_pack(row_nlse, row_nlse);
            ndel2 = f2_pack(row_ndelta, row_ndelta);
          } else {
            const float4 sv = stats4[c >> 1];
            nlse2 = f2_pack(sv.x, sv.y);
            ndel2 = f2_pack(sv.z, sv.w);
          }
          // p = exp2(s * qk_scale - lse * log2e) for two columns at once
          float x_a, x_b;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(t1[c]), __uint_as_float(t1[c + 1])), scale2, nlse2), x_a, x_b);
          float p_a = fast_exp2(x_a);
          float p_b = fast_exp2(x_b);
          if constexpr (DIAG) {
            bool vis_a, vis_b;
            if constexpr (MODE == MODE_Q) {
              const int d = row + P_SEQ - (col0 + c);
              vis_a = d >= my_d_min && d < my_d_max;
              vis_b = d - 1 >= my_d_min && d - 1 < my_d_max;
            } else {
              const int d = col0 + c + P_SEQ - row;
              vis_a = d >= my_d_min && d < my_d_max;
              vis_b = d + 1 >= my_d_min && d + 1 < my_d_max;
            }
            p_a = vis_a ? p_a : 0.f;
            p_b = vis_b ? p_b : 0.f;
          }
          if constexpr (MODE == MODE_TOTAL) {
            tot_sum += p_a + p_b;
          } else {
            float dp_a = __uint_as_float(t2[c]);
            float dp_b = __uint_as_float(t2[c + 1]);
            float pd_a = p_a, pd_b = p_b;
            if constexpr (DROPOUT) {
              const bool keep_a = (keep_bits >> c) & 1u;
              const bool keep_b = (keep_bits >> (c + 1)) & 1u;
              pd_a = keep_a ? p_a : 0.f;
              pd_b = keep_b ? p_b : 0.f;
              dp_a = keep_a ? dp_a * args.drop.inv_keep : 0.f;
              dp_b = keep_b ? dp_b * args.drop.inv_keep : 0.f;
            }
            // dS = P * (dP - delta)
            float ds_a, ds_b;
            f2_unpack(f2_mul(f2_pack(p_a, p_b), f2_add(f2_pack(dp_a, dp_b), ndel2)), ds_a, ds_b);
            t1[c >> 1] = pack2<BF16>(pd_a, pd_b);
            t2[c >> 1] = pack2<BF16>(ds_a, ds_b);
          }
        }
      };
      if (diag) recompute(std::true_type{}); else recompute(std::false_type{});
      if constexpr (MODE != MODE_TOTAL) {
        // Outputs go over this group's own (already loaded) T1 columns only, so the two groups
        // never touch each other's unread inputs.
        if constexpr (MODE == MODE_KV) tmem_st16(t1_addr + wg * HALF, t1);
        tmem_st16(t1_addr + wg * HALF + 16, t2);
        if constexpr (FUSED) {
          // dS^T once more, as the shared-memory B operand of dQ^T: row = key, 64 queries = 128
          // bytes, 16-byte chunks permuted by the 128-byte swizzle.
          // (one tile: the product that read the previous step's copy must have completed)
          if (i >= 1) {
            const bool w = wait(&dq_ready[dq_slot(i - 1)], dq_phase(i - 1));
            if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_MMA); ok = false; break; }
          }
          uint8_t* ds_row = sDS + row_local * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int chunk = (wg * 4 + j) ^ (row_local & 7);
            *reinterpret_cast<uint4*>(ds_row + chunk * 16) =
                make_uint4(t2[4 * j + 0], t2[4 * j + 1], t2[4 * j + 2], t2[4 * j + 3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(&p_ready[buf]);
    }

    // ------------------------------------------------------------- epilogue
    if (ok && T > 0) {
      const bool w = wait(acc_full, 0);
      if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_MMA); ok = false; }
    }
    if constexpr (MODE == MODE_TOTAL) {
      // The two groups hold partial sums of alternating steps: combine through shared memory.
      float* red = reinterpret_cast<float*>(sA);  // the resident tile is dead after acc_full
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (wg == 1) red[row_local] = tot_sum;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (wg == 0 && ok && row < args.N)
        args.tot[(static_cast<int64_t>(b) * args.Hq + h_first) * args.N + row] = tot_sum + red[row_local];
    } else if (args.out_tma) {
      // Each thread scales and rounds its half row of every accumulator into the (now dead) resident
      // tile of the same index, in the swizzled layout of the output tensor map; one thread then
      // stores the 128 x D tiles with TMA, which clips rows past the end of the tensor. (Storing from
      // registers, below, writes 32 rows x 16 bytes per warp instruction and takes several
      // microseconds per CTA.) Warps that gave up still come to the meeting point.
      tc_fence_after();
      const int out_head = MODE == MODE_Q ? h_first : hk;
      constexpr int NC = D / 2;  // columns per thread and accumulator
#pragma unroll
      for (int acc = 0; acc < N_ACC; ++acc) {
        float scale = args.sm_scale;
        if (MODE == MODE_KV && acc == 1) scale = DROPOUT ? args.drop.inv_keep : 1.0f;
        uint32_t o[NC];
        if (T > 0 && ok) {
#pragma unroll
          for (int x = 0; x < NC; x += 8) {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                : "=r"(o[x + 0]), "=r"(o[x + 1]), "=r"(o[x + 2]), "=r"(o[x + 3]), "=r"(o[x + 4]), "=r"(o[x + 5]),
                  "=r"(o[x + 6]), "=r"(o[x + 7])
                : "r"(tmem_base + lane_base + acc * D + wg * NC + x)
                : "memory");
          }
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < NC; ++i) o[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < NC; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * scale);
        if constexpr (MODE == MODE_KV) {
          // dV on top of a gradient that is already there (second region of piecewise attention):
          // added in fp32, rounded once.
          if (acc == 1 && args.out2_accumulate && row < args.N) {
            const uint16_t* prev = static_cast<const uint16_t*>(args.out2) + b * args.out2_sb + hk * args.out2_sh +
                                   static_cast<int64_t>(row) * args.out2_sr + wg * NC;
#pragma unroll
            for (int x = 0; x < NC; x += 8) {
              const uint4 pv = *reinterpret_cast<const uint4*>(prev + x);
              const uint32_t w[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = unpack2<BF16>(w[i]);
                o[x + 2 * i] = __float_as_uint(__uint_as_float(o[x + 2 * i]) + f.x);
                o[x + 2 * i + 1] = __float_as_uint(__uint_as_float(o[x + 2 * i + 1]) + f.y);
              }
            }
          }
        }
        const uint32_t tile = smem_u32(sA + acc * Cfg::TILE_BYTES);
#pragma unroll
        for (int x = 0; x < NC; x += 8) {
          const int c = wg * NC + x;  // first of 8 columns = one 16-byte unit
          const uint32_t row_addr = tile + (c / Cfg::CHUNK) * Cfg::CHUNK_BYTES + row_local * Cfg::ROW_BYTES;
          const uint32_t swz = (row_addr >> 7) & (Cfg::ROW_BYTES / 16 - 1);
          const uint32_t dst = row_addr + (((static_cast<uint32_t>(c % Cfg::CHUNK) >> 3) ^ swz) << 4);
          const uint32_t v0 = pack2<BF16>(__uint_as_float(o[x + 0]), __uint_as_float(o[x + 1]));
          const uint32_t v1 = pack2<BF16>(__uint_as_float(o[x + 2]), __uint_as_float(o[x + 3]));
          const uint32_t v2 = pack2<BF16>(__uint_as_float(o[x + 4]), __uint_as_float(o[x + 5]));
          const uint32_t v3 = pack2<BF16>(__uint_as_float(o[x + 6]), __uint_as_float(o[x + 7]));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                       : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_sync);
      if (warp == 0) {
        const bool w = wait(epi_sync, 0);
        if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_SOFTMAX); ok = false; }
        if (ok && lane == 0 && !*abort_flag) {
#pragma unroll
          for (int acc = 0; acc < N_ACC; ++acc) {
#pragma unroll
            for (int ch = 0; ch < Cfg::NCHUNK; ++ch)
              tma_store_4d(acc == 0 ? &tmO1 : &tmO2, sA + acc * Cfg::TILE_BYTES + ch * Cfg::CHUNK_BYTES,
                           ch * Cfg::CHUNK, r0, out_head, b);
          }
          tma_store_commit();
          tma_store_wait_all();  // shared memory must outlive the reads of the stores
        }
      }
    } else if (ok) {
      tc_fence_after();
      const int n_rows = MODE == MODE_Q ? args.M : args.N;
      const bool valid = row < n_rows;
      const int out_head = MODE == MODE_Q ? h_first : hk;
      // Group `wg` converts half of the columns of every accumulator.
#pragma unroll
      for (int acc = 0; acc < N_ACC; ++acc) {
        void* out = acc == 0 ? args.out1 : args.out2;
        const int64_t off = acc == 0
                                ? b * args.out1_sb + out_head * args.out1_sh + static_cast<int64_t>(row) * args.out1_sr
                                : b * args.out2_sb + out_head * args.out2_sh + static_cast<int64_t>(row) * args.out2_sr;
        float scale = args.sm_scale;
        if (MODE == MODE_KV && acc == 1) scale = DROPOUT ? args.drop.inv_keep : 1.0f;
#pragma unroll
        for (int c = wg * (D / 2); c < (wg + 1) * (D / 2); c += 8) {
          uint32_t o[8];
          __syncwarp();
          if (T > 0) {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]),
                  "=r"(o[7])
                : "r"(tmem_base + lane_base + acc * D + c)
                : "memory");
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = 0u;
          }
          if (valid) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[i]) * scale;
            if (MODE == MODE_KV && acc == 1 && args.out2_accumulate) {
              const uint4 pv = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(out) + off + c);
              const uint32_t w[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 g = unpack2<BF16>(w[i]);
                f[2 * i] += g.x;
                f[2 * i + 1] += g.y;
              }
            }
            uint4 v;
            v.x = pack2<BF16>(f[0], f[1]);
            v.y = pack2<BF16>(f[2], f[3]);
            v.z = pack2<BF16>(f[4], f[5]);
            v.w = pack2<BF16>(f[6], f[7]);
            *reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + off + c) = v;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  __syncwarp();
  if (warp == 8) {
    if (*abort_flag) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {}
    }
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200attn
