// Forward attention kernel for sm_100a.
//
// A work item is 256 query rows of one (batch, head): two 128-row tiles that share every
// K/V tile brought into shared memory. Roles of a CTA:
//   warps 0-3  : softmax + epilogue for query tile 0 (thread r <-> row r, TMEM lane r)
//   warps 4-7  : softmax + epilogue for query tile 1
//   warp 8     : tcgen05.mma issuer (one elected lane)
//   warp 9     : TMA producer (one elected lane); warp 10 takes the V ring of a paged cache;
//                warps 10-11 are otherwise idle (they complete the third warpgroup so that
//                registers can be moved to the softmax groups)
// TMEM (512 columns): S0 | S1 (128 fp32 columns each, P aliases the first 64 columns of its S
// as packed 16-bit pairs) and O0 | O1 (D fp32 columns each).
// The two tiles ping-pong: while one tile's softmax runs on the CUDA cores the tensor core
// executes the other tile's GEMMs.
//
// The grid may hold fewer CTAs than work items (one CTA per SM): every role then walks the same
// list of items, the barrier phases and the K/V ring position carry over from one item to the next,
// and the loads of the next item's Q and first K/V tiles are issued while the current item's last
// softmax and epilogue still run, so TMEM allocation, barrier set-up, the first load latency and the
// output stores of one item hide behind the work of its neighbours.
//
// Numerics follow the reference kernel (flash.py:442-509): S = QK^T with fp32 accumulation,
// base-2 online softmax with qk_scale = sm_scale*log2(e), the row sum taken before dropout and
// before P is rounded to the input type, O normalised once at the end, LSE = m*sm_scale + ln(l).
// The running maximum is only raised when it grows by more than 2^8 (the accumulators are
// rescaled then), which leaves O and LSE unchanged up to fp32 rounding.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace b200attn {

template <int D>
struct TileCfg {
  static constexpr int BLOCK = 128;                       // rows of a Q tile / a K,V tile
  static constexpr int CHUNK = D >= 64 ? 64 : D;          // elements per swizzled row segment
  static constexpr int NCHUNK = D / CHUNK;
  static constexpr int ROW_BYTES = CHUNK * 2;             // 128 / 64 / 32
  static constexpr uint32_t UMMA_SWZ = ROW_BYTES == 128 ? SWZ_128B : (ROW_BYTES == 64 ? SWZ_64B : SWZ_32B);
  static constexpr int TMA_SWZ = ROW_BYTES == 128 ? 3 : (ROW_BYTES == 64 ? 2 : 1);
  static constexpr int CHUNK_BYTES = BLOCK * ROW_BYTES;   // one [128 x CHUNK] box
  static constexpr int TILE_BYTES = BLOCK * D * 2;
  static constexpr int STEPS_PER_CHUNK = CHUNK / 16;
  // K-major operand (rows = M or N of the MMA, contiguous along the contraction).
  static constexpr uint64_t KMAJOR_DESC = make_smem_desc_hi(16, 8 * ROW_BYTES, UMMA_SWZ);
  // MN-major operand (rows = contraction index, contiguous along the MMA's N).
  static constexpr uint64_t MNMAJOR_DESC = make_smem_desc_hi(CHUNK_BYTES, 8 * ROW_BYTES, UMMA_SWZ);
};

struct FwdArgs {
  void* o;
  float* lse;
  int64_t o_stride_b, o_stride_h, o_stride_m, o_stride_split;
  int64_t lse_stride_b, lse_stride_h, lse_stride_split;
  int n_zblocks, grid_chunk;        // work-item order, see decode_block()
  BlockOrder order;                 // the same order with its divisions prepared on the host
  FastDiv div_heads, div_groups, div_splits;  // by the heads of the item grid, groups, num_splits
  int o_tma;                        // the output goes through shared memory and TMA stores (16-bit O only)
  int n_items;                      // number of work items; with fewer CTAs than items CTA c of G takes
                                    // items c, 2G-1-c, 2G+c, 4G-1-c, ... (the items are sorted from long
                                    // to short, so this back-and-forth order evens out the CTAs' totals).
                                    // Only the plain mode (no packing, one split, dense K/V) may do so.
  int num_splits, tiles_per_split;  // split-KV: CTA `split` visits K/V tiles [split*tps, (split+1)*tps)
  int pack_heads;                   // > 0: decode-style packing, the CTA's tile 0 holds all `groups`
                                    // query heads of one KV head (rows = head-major, M rows each,
                                    // groups * M <= 128) so K/V are streamed once per KV head
  int dual_stream;                  // with pack_heads: tile 1 holds the same rows as tile 0 and the two
                                    // tiles take alternate K/V tiles of the CTA's key range, as two
                                    // independent softmax chains; tile t writes partial 2 * split + t
  int ring_stages;                  // dual_stream: K/V ring depth (one shared Q tile leaves room for more)
  // Paged K/V (block_table != nullptr): the K and V tensor maps describe caches [num_blocks, Hkv,
  // block, D] with boxes of min(block, 128) rows; key n of sequence b lives in block
  // block_table[b * bt_stride + (n >> block_shift)] at row n & (block - 1), and the sequence's
  // key count comes from context_lens[b] instead of N.
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* context_lens;
  int block_shift;
  int B, Hq, Hkv, M, N, groups;
  int causal, o_fp32;               // causal: some band limit below is finite (enables the masking code)
  // Visibility band: query m sees key n iff d_min <= m + (N - M) - n < d_max. Plain causal masking is
  // d_min = 0; no mask is (-BAND_INF, BAND_INF); a sliding window or the two regions of piecewise
  // attention set both.
  int d_min, d_max;
  float sm_scale, qk_scale;
  DropoutCtx drop;
  int32_t* status;
};

template <int D>
struct FwdSmem {
  static constexpr int STAGES = D == 128 ? 2 : (D == 64 ? 3 : 4);
  static constexpr int Q_BYTES = 2 * TileCfg<D>::TILE_BYTES;
  static constexpr int KV_BYTES = STAGES * TileCfg<D>::TILE_BYTES;
  // Output staging for the TMA stores: one [128 x CHUNK] box per query tile.
  static constexpr int O_STAGE_BYTES = 2 * TileCfg<D>::CHUNK_BYTES;
  static constexpr int BAR_OFFSET = Q_BYTES + 2 * KV_BYTES + O_STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 512 + 1024;  // barriers + alignment slack
  // Dual-stream mode: one Q tile, as deep a ring as fits (at most 8 stages: the barrier block
  // holds 18 + 4 * stages barriers in 512 bytes).
  static constexpr int MAX_TOTAL = 232448;
  static constexpr int DUAL_STAGES_FIT = (MAX_TOTAL - 1536 - TileCfg<D>::TILE_BYTES) / (2 * TileCfg<D>::TILE_BYTES);
  static constexpr int DUAL_STAGES = DUAL_STAGES_FIT > 8 ? 8 : DUAL_STAGES_FIT;
  static constexpr int DUAL_TOTAL = (1 + 2 * DUAL_STAGES) * TileCfg<D>::TILE_BYTES + 512 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

static constexpr float RESCALE_THRESHOLD = 8.0f;
static constexpr int BAND_INF = 1 << 30;

// Which of every 8 consecutive column pairs compute their exponential with the polynomial on the
// FMA pipe instead of ex2.approx on the special-function unit (bit k = pair k). The smaller the head
// dimension, the fewer tensor-core cycles stand against the 16-per-clock special-function unit, so
// the larger the share that pays.
#ifndef B200ATTN_FWD_POLY_MASK_D128
#define B200ATTN_FWD_POLY_MASK_D128 0x00u
#endif
#ifndef B200ATTN_FWD_POLY_MASK_SMALL_D
#define B200ATTN_FWD_POLY_MASK_SMALL_D 0x11u
#endif
template <int D>
struct PolyMask {
  static constexpr uint32_t value = D >= 128 ? B200ATTN_FWD_POLY_MASK_D128 : B200ATTN_FWD_POLY_MASK_SMALL_D;
};

// SPLIT64 (D = 128, plain mode only: no head packing, no paged cache): the softmax works on 64 keys at a
// time and each query tile's 128 S columns hold two 64-key score buffers, so Q K^T of sub-step u + 2 is
// issued right behind P V of sub-step u and is complete long before the softmax group has finished
// sub-step u + 1: the group never waits for its own tile's tensor-core work (with one 128-column S per
// tile, as below, softmax -> P V -> next Q K^T -> softmax of one tile are strictly serial and the tensor
// pipe idles while a tile's softmax runs). P of a sub-step overwrites the first 32 columns of its own
// buffer. The accumulator is no longer quiescent while a softmax step runs, so the (rare) rescale of
// O first waits on `pv_done` for the previous sub-step's P V.
template <int D, bool BF16, bool DROPOUT, bool SPLIT64 = false>
__global__ void __launch_bounds__(384, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
           const FwdArgs args) {
  using Cfg = TileCfg<D>;
  using Sm = FwdSmem<D>;
  constexpr int STAGES = Sm::STAGES;
  constexpr int BLOCK = Cfg::BLOCK;
  constexpr int SUB = 64;  // SPLIT64: keys per softmax sub-step
  static_assert(!SPLIT64 || D == 128, "the 64-key pipeline exists for D = 128");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  // Layout: Q tiles | K ring | V ring | output staging | barriers. The dual-stream mode keeps one Q
  // tile (both query tiles hold the same rows), no output staging (its partial outputs are fp32 and
  // stored directly) and spends the space on a deeper ring.
  const bool dual = args.pack_heads > 0 && args.dual_stream != 0;
  // SPLIT64: the same ring memory holds twice as many slots of 64 keys each, so that a slot is
  // reloaded four sub-steps before its next use (with whole 128-key tiles in two slots the loads of
  // the faster pipeline arrive late).
  constexpr int SLOT_BYTES = SPLIT64 ? Cfg::TILE_BYTES / 2 : Cfg::TILE_BYTES;
  constexpr int SLOT_CHUNK_BYTES = SPLIT64 ? Cfg::CHUNK_BYTES / 2 : Cfg::CHUNK_BYTES;  // one [rows x CHUNK] box
  const int stages = dual ? args.ring_stages : (SPLIT64 ? 2 * STAGES : STAGES);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + (dual ? 1 : 2) * Cfg::TILE_BYTES;
  uint8_t* sV = sK + stages * SLOT_BYTES;
  uint8_t* sO = sV + stages * SLOT_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sO + (dual ? 0 : Sm::O_STAGE_BYTES));
  uint64_t* q_full = bars;                  // [2]
  uint64_t* k_full = bars + 2;              // [stages]
  uint64_t* k_empty = k_full + stages;      // [stages]
  uint64_t* v_full = k_empty + stages;      // [stages]
  uint64_t* v_empty = v_full + stages;      // [stages]
  uint64_t* s_full = v_empty + stages;      // [2] (SPLIT64: [2 tiles][2 buffers])
  uint64_t* p_half = s_full + 4;            // [2 tiles][2 halves] (SPLIT64: P of buffer 0 / 1)
  uint64_t* o_full = p_half + 4;            // [2]
  uint64_t* q_empty = o_full + 2;           // [2]
  uint64_t* pv_done = q_empty + 2;          // [2] SPLIT64: every P V issued so far for the tile has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool packed = args.pack_heads > 0;
  const int grid_heads = packed ? args.Hkv : args.Hq;
  const bool paged = args.block_table != nullptr;

  // One work item: 256 query rows of one (batch, head) and, with split K/V, one range of keys.
  struct Item {
    int b, hk, h, m0, split, N_ctx, P_SEQ;
    int j0;          // first K/V tile the CTA streams
    int n_tiles[2];  // number of K/V tiles each query tile visits
    int n_sub[2];    // SPLIT64: number of 64-key sub-steps each query tile runs
    int n_max;       // number of K/V tiles the CTA streams
  };
  auto get_item = [&](int id) -> Item {
    Item it;
    const BlockCoord bc = args.order.decode(id);
    const int z_row = args.div_splits.div(bc.z);
    it.split = bc.z - z_row * args.num_splits;
    const int m_blk = args.div_splits.div(args.n_zblocks) - 1 - z_row;  // longest first
    const int j_split = it.split * args.tiles_per_split;  // first K/V tile of this item's split
    it.b = args.div_heads.div(bc.bh);
    const int head = bc.bh - it.b * grid_heads;
    it.hk = packed ? head : args.div_groups.div(head);
    it.h = packed ? it.hk * args.groups : head;   // first (or only) query head
    it.m0 = m_blk * 2 * BLOCK;
    it.N_ctx = paged ? args.context_lens[it.b] : args.N;
    it.P_SEQ = it.N_ctx - args.M;
    // First K/V tile: the split's first tile, or the first tile that the band's far edge lets the
    // item's first query row see (the second query tile then meets one fully masked tile first,
    // which costs one iteration).
    it.j0 = j_split;
    if (args.causal && args.d_max < BAND_INF) it.j0 = max(it.j0, max(0, it.m0 + it.P_SEQ - args.d_max + 1) / BLOCK);
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int mt = it.m0 + t * BLOCK;
      int hi = it.N_ctx;
      if (args.causal && args.d_min > -BAND_INF) hi = min(it.N_ctx, max(0, it.P_SEQ + mt + BLOCK - args.d_min));
      int n_full = mt < args.M ? cdiv(hi, BLOCK) : 0;
      if (packed) {
        // one tile holds every row of every head of the group: rows m = 0..M-1
        const int hi_p = (args.causal && args.d_min > -BAND_INF) ? min(it.N_ctx, max(0, it.P_SEQ + args.M - args.d_min)) : it.N_ctx;
        n_full = t == 0 ? cdiv(hi_p, BLOCK) : 0;
      }
      it.n_tiles[t] = max(0, min(n_full, j_split + args.tiles_per_split) - it.j0);
      // (a last half tile that no row of the query tile sees is not computed)
      it.n_sub[t] = mt < args.M ? max(0, cdiv(min(hi, (j_split + args.tiles_per_split) * BLOCK), SUB) - 2 * it.j0) : 0;
      if constexpr (SPLIT64) it.n_tiles[t] = (it.n_sub[t] + 1) / 2;
    }
    if (dual) {
      const int n = it.n_tiles[0];
      it.n_tiles[0] = (n + 1) / 2;
      it.n_tiles[1] = n / 2;
    }
    it.n_max = dual ? it.n_tiles[0] + it.n_tiles[1] : max(it.n_tiles[0], it.n_tiles[1]);
    return it;
  };
  // Item of this CTA's k-th round (see FwdArgs::n_items); out of range ends the CTA's list.
  auto item_of_round = [&](int k) -> int {
    const int G = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
    return k * G + ((k & 1) ? G - 1 - c : c);
  };

  if (threadIdx.x == 0) {
    mbar_init(&q_full[0], 1);
    mbar_init(&q_full[1], 1);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], SPLIT64 ? 2 : 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], SPLIT64 ? 2 : 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&s_full[2 + t], 1);
      mbar_init(&pv_done[t], 1);
      mbar_init(&p_half[2 * t], 128);
      mbar_init(&p_half[2 * t + 1], 128);
      mbar_init(&o_full[t], 1);
      mbar_init(&q_empty[t], 1);
    }
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

  if (warp == 11) {
    reg_dealloc<80>();
  } else if (warp == 9 || (!SPLIT64 && warp == 10)) {
    // ------------------------------------------------------------ TMA producers
    // Warp 9 loads Q and streams the K and V tiles (one elected lane). With a paged cache a tile is
    // up to 16 small copies per operand and one thread cannot issue them fast enough, so warp 10
    // then takes the V ring (each ring has its own barriers).
    reg_dealloc<80>();
    if (lane == 0 && (warp == 9 || paged)) {
      if (warp == 9) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
      }
      // Ring position and barrier phases run on from one work item to the next.
      int st = 0;
      uint32_t par = 1;            // first pass over the ring passes at once
      uint32_t q_par[2] = {1, 1};  // and so does the first use of each Q tile
      bool alive = true;
      for (int k = 0; alive; ++k) {
        const int id = item_of_round(k);
        if (id >= args.n_items || (k > 0 && *abort_flag)) break;
        const Item it = get_item(id);
        if (it.n_max == 0) continue;
        if (warp == 9) {
          for (int t = 0; t < (dual ? 1 : 2); ++t) {
            if (it.n_tiles[t] == 0) continue;
            // the previous item's last Q K^T on this tile has read the buffer
            if (!wait(&q_empty[t], q_par[t])) { fail(ST_WAIT_EMPTY); alive = false; break; }
            q_par[t] ^= 1;
            // packed: the box is [groups heads x M rows x CHUNK], landing head-major in the tile
            mbar_expect_tx(&q_full[t], packed ? args.groups * args.M * D * 2 : Cfg::TILE_BYTES);
            for (int c = 0; c < Cfg::NCHUNK; ++c)
              tma_load_4d(sQ + t * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmQ, &q_full[t],
                          c * Cfg::CHUNK, packed ? 0 : it.m0 + t * BLOCK, it.h, it.b);
          }
          if (!alive) break;
        }
        if constexpr (SPLIT64) {
          // Ring position i of an item holds the keys of sub-step i in its K slot and the values of
          // sub-step i - 2 in its V slot (Q K^T of sub-step u + 2 is issued together with P V of
          // sub-step u), behind one pair of barriers (k_full / k_empty). The position runs on across items.
          const int n_sub_max = max(it.n_sub[0], it.n_sub[1]);
          const int key0 = it.j0 * BLOCK;
          for (int i = 0; i < n_sub_max + 2 && alive; ++i) {
            const bool has_k = i < n_sub_max, has_v = i >= 2;
            if (!has_k && !has_v) continue;
            if (st == stages) { st = 0; par ^= 1; }
            if (!wait(&k_empty[st], par)) { fail(ST_WAIT_EMPTY); alive = false; break; }
            mbar_expect_tx(&k_full[st], (has_k ? SLOT_BYTES : 0) + (has_v ? SLOT_BYTES : 0));
            if (has_k) {
              for (int c = 0; c < Cfg::NCHUNK; ++c)
                tma_load_4d(sK + st * SLOT_BYTES + c * SLOT_CHUNK_BYTES, &tmK, &k_full[st],
                            c * Cfg::CHUNK, key0 + i * SUB, it.hk, it.b);
            }
            if (has_v) {
              for (int c = 0; c < Cfg::NCHUNK; ++c)
                tma_load_4d(sV + st * SLOT_BYTES + c * SLOT_CHUNK_BYTES, &tmV, &k_full[st],
                            c * Cfg::CHUNK, key0 + (i - 2) * SUB, it.hk, it.b);
            }
            ++st;
          }
        } else if (!paged) {
          // Dense K/V: one tile = 128 consecutive keys = one box per 64-column chunk.
          for (int j = 0; j < it.n_max; ++j, ++st) {
            if (st == stages) { st = 0; par ^= 1; }
            if (!wait(&k_empty[st], par)) { fail(ST_WAIT_EMPTY); alive = false; break; }
            mbar_expect_tx(&k_full[st], Cfg::TILE_BYTES);
            for (int c = 0; c < Cfg::NCHUNK; ++c)
              tma_load_4d(sK + st * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmK, &k_full[st],
                          c * Cfg::CHUNK, (it.j0 + j) * BLOCK, it.hk, it.b);
            if (!wait(&v_empty[st], par)) { fail(ST_WAIT_EMPTY); alive = false; break; }
            mbar_expect_tx(&v_full[st], Cfg::TILE_BYTES);
            for (int c = 0; c < Cfg::NCHUNK; ++c)
              tma_load_4d(sV + st * Cfg::TILE_BYTES + c * Cfg::CHUNK_BYTES, &tmV, &v_full[st],
                          c * Cfg::CHUNK, (it.j0 + j) * BLOCK, it.hk, it.b);
          }
        } else {
          // Paged K/V: the tile spans 128 / block cache blocks, one box per block and chunk. Boxes past
          // the sequence's last block re-read that block, so the tile holds defined data everywhere
          // (those keys are masked, and stale V rows are cleared before use).
          const bool k_side = warp == 9;
          const CUtensorMap* tm = k_side ? &tmK : &tmV;
          uint8_t* ring = k_side ? sK : sV;
          uint64_t* full = k_side ? k_full : v_full;
          uint64_t* empty = k_side ? k_empty : v_empty;
          const int block = 1 << args.block_shift;
          const int box_rows = min(block, BLOCK);
          const int last_blk = (it.N_ctx - 1) >> args.block_shift;
          for (int j = 0; j < it.n_max; ++j, ++st) {
            if (st == stages) { st = 0; par ^= 1; }
            if (!wait(&empty[st], par)) { fail(ST_WAIT_EMPTY); alive = false; break; }
            uint8_t* dst = ring + st * Cfg::TILE_BYTES;
            mbar_expect_tx(&full[st], Cfg::TILE_BYTES);
            for (int r = 0; r < BLOCK; r += box_rows) {
              const int n_start = (it.j0 + j) * BLOCK + r;
              const int blk = args.block_table[it.b * args.bt_stride + min(n_start >> args.block_shift, last_blk)];
              for (int c = 0; c < Cfg::NCHUNK; ++c)
                tma_load_4d(dst + c * Cfg::CHUNK_BYTES + r * Cfg::ROW_BYTES, tm, &full[st], c * Cfg::CHUNK,
                            n_start & (block - 1), it.hk, blk);
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 8 || (SPLIT64 && warp == 10)) {
    // ------------------------------------------------------------- MMA issuer
    // (SPLIT64: one issuing warp per query tile, warp 8 for tile 0 and warp 10 for tile 1)
    // The whole warp runs this loop with warp-uniform values; one elected lane issues each
    // tcgen05 instruction (see mma_ss_w).
    reg_dealloc<80>();
    constexpr uint32_t IDESC_QK = make_idesc(BF16, 128, BLOCK, false, false);
    constexpr uint32_t IDESC_PV = make_idesc(BF16, 128, D, false, true);
    const uint32_t q_addr = smem_u32(sQ);
    const uint32_t k_addr = smem_u32(sK);
    const uint32_t v_addr = smem_u32(sV);
    auto issue_qk = [&](int t, int st) {
      const uint64_t dq = smem_desc(Cfg::KMAJOR_DESC, q_addr + (dual ? 0 : t) * Cfg::TILE_BYTES);
      const uint64_t dk = smem_desc(Cfg::KMAJOR_DESC, k_addr + st * Cfg::TILE_BYTES);
#pragma unroll
      for (int s = 0; s < D / 16; ++s) {
        // offsets are multiples of 16 bytes inside shared memory: they add into the 14-bit
        // address field of the descriptor without carrying out of it
        const uint32_t off = ((s / Cfg::STEPS_PER_CHUNK) * Cfg::CHUNK_BYTES +
                              (s % Cfg::STEPS_PER_CHUNK) * 32) >> 4;
        mma_ss_w(tmem_base + t * BLOCK, dq + off, dk + off, IDESC_QK, s > 0 ? 1u : 0u);
      }
    };
    // SPLIT64: S buffer h of tile t (64 fp32 columns) = Q_t x (keys 64 h .. 64 h + 63 of the K tile)^T
    // SPLIT64: S buffer h of tile t (64 fp32 columns) = Q_t x (the 64 keys in K slot `st`)^T
    auto issue_qk64 = [&](int t, int st, int h) {
      constexpr uint32_t IDESC_QK64 = make_idesc(BF16, 128, SUB, false, false);
      const uint64_t dq = smem_desc(Cfg::KMAJOR_DESC, q_addr + t * Cfg::TILE_BYTES);
      const uint64_t dk = smem_desc(Cfg::KMAJOR_DESC, k_addr + st * SLOT_BYTES);
#pragma unroll
      for (int s = 0; s < D / 16; ++s) {
        const uint32_t off_q = ((s / Cfg::STEPS_PER_CHUNK) * Cfg::CHUNK_BYTES + (s % Cfg::STEPS_PER_CHUNK) * 32) >> 4;
        const uint32_t off_k = ((s / Cfg::STEPS_PER_CHUNK) * SLOT_CHUNK_BYTES + (s % Cfg::STEPS_PER_CHUNK) * 32) >> 4;
        mma_ss_w(tmem_base + t * BLOCK + h * SUB, dq + off_q, dk + off_k, IDESC_QK64, s > 0 ? 1u : 0u);
      }
    };
    // SPLIT64: O_t (+)= P (the first 32 columns of buffer h) x the 64 keys in V slot `st`
    auto issue_pv64 = [&](int t, int st, bool acc, int h) {
      constexpr uint64_t V_DESC = make_smem_desc_hi(SLOT_CHUNK_BYTES, 8 * Cfg::ROW_BYTES, Cfg::UMMA_SWZ);
      const uint64_t dv = smem_desc(V_DESC, v_addr + st * SLOT_BYTES);
#pragma unroll
      for (int s = 0; s < SUB / 16; ++s) {
        mma_ts_w(tmem_base + 2 * BLOCK + t * D, tmem_base + t * BLOCK + h * SUB + s * 8,
                 dv + ((s * 16 * Cfg::ROW_BYTES) >> 4), IDESC_PV, (acc || s > 0) ? 1u : 0u);
      }
    };
    auto issue_pv = [&](int t, int st, bool acc, int half) {
      const uint64_t dv = smem_desc(Cfg::MNMAJOR_DESC, v_addr + st * Cfg::TILE_BYTES);
#pragma unroll
      for (int s = half * (BLOCK / 32); s < (half + 1) * (BLOCK / 32); ++s) {
        mma_ts_w(tmem_base + 2 * BLOCK + t * D, tmem_base + t * BLOCK + s * 8,
                 dv + ((s * 16 * Cfg::ROW_BYTES) >> 4), IDESC_PV, (acc || s > 0) ? 1u : 0u);
      }
    };
    // Paged caches only: the last block of a sequence holds rows past its context length whose
    // contents are arbitrary. Their probabilities are exactly zero, but 0 x NaN is NaN in the
    // product, so those V rows are cleared in shared memory before P V reads them.
    // (first_bad: the first row of the tile in ring slot st that lies past the context length)
    auto clear_stale_v_rows = [&](int st, int first_bad) {
      if (!paged) return;
      if (first_bad >= BLOCK) return;
      uint8_t* tile = sV + st * Cfg::TILE_BYTES;
      for (int r = max(first_bad, 0) + lane; r < BLOCK; r += 32) {
        for (int c = 0; c < Cfg::NCHUNK; ++c) {
          uint4* row = reinterpret_cast<uint4*>(tile + c * Cfg::CHUNK_BYTES + r * Cfg::ROW_BYTES);
#pragma unroll
          for (int k = 0; k < Cfg::ROW_BYTES / 16; ++k) row[k] = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
    };
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int32_t code) -> bool {
      const bool w = wait(bar, parity);
      if (__all_sync(0xffffffffu, w)) return true;
      fail(code);
      return false;
    };
    // Ring slot and phase of the current K/V tile, and the phases of the per-tile barriers: all of
    // them run on from one work item to the next.
    int st = 0;
    uint32_t ph = 0;
    uint32_t q_ph[2] = {0, 0}, p_ph[2] = {0, 0};
    uint32_t p_ph_b[2] = {0, 0};       // SPLIT64: phases of the second score buffer's P barriers (p_ph: the first)
    int ks = 0;                        // SPLIT64: ring position of the next sub-step
    uint32_t kph = 0;
    for (int k = 0;; ++k) {
      const int id = item_of_round(k);
      if (id >= args.n_items || (k > 0 && *abort_flag)) break;
      const Item it = get_item(id);
      if (it.n_max == 0) continue;
      const int n_max = it.n_max;
      if constexpr (SPLIT64) {
        // Sub-step u of a query tile works on keys [64 u, 64 u + 64) of the item's key range, score
        // buffer u & 1; K slot ks holds the keys of sub-step u + 2 while V slot vs holds those of
        // sub-step u. Issue order per sub-step and query tile: P V (u), then Q K^T (u + 2) into the
        // buffer that P V just freed.
        const int n_sub_max = max(it.n_sub[0], it.n_sub[1]);
        const int t = warp == 8 ? 0 : 1;   // this warp's query tile
        const int n_mine = it.n_sub[t];
        bool ok = true;
        // Ring positions 0 and 1 hold only keys: the first two Q K^T.
#pragma unroll
        for (int u0 = 0; u0 < 2; ++u0) {
          if (!ok || u0 >= n_sub_max) break;
          // (every position is awaited before it is released, with or without work on it: a warp whose
          // tile has nothing to do must not run ahead of the other by a whole pass over the ring)
          if (!wait_all(&k_full[ks], kph, ST_WAIT_TMA)) { ok = false; break; }
          if (u0 < n_mine) {
            if (u0 == 0) {
              if (!wait_all(&q_full[t], q_ph[t], ST_WAIT_TMA)) { ok = false; break; }
              q_ph[t] ^= 1;
            }
            tc_fence_after();
            issue_qk64(t, ks, u0);
            tc_commit_w(&s_full[2 * t + u0]);
            if (u0 + 1 == n_mine) tc_commit_w(&q_empty[t]);  // the item's last read of Q_t
          }
          tc_commit_w(&k_empty[ks]);
          if (++ks == stages) { ks = 0; kph ^= 1u; }
        }
        // Position of sub-step u: values of sub-step u and keys of sub-step u + 2.
        for (int u = 0; u < n_sub_max && ok; ++u) {
          const int h = u & 1;
          if (!wait_all(&k_full[ks], kph, ST_WAIT_TMA)) { ok = false; break; }
          if (u < n_mine) {
            if (!wait_all(&p_half[2 * t + h], h ? p_ph_b[t] : p_ph[t], ST_WAIT_SOFTMAX)) { ok = false; break; }
            if (h) p_ph_b[t] ^= 1; else p_ph[t] ^= 1;
            tc_fence_after();
            issue_pv64(t, ks, u > 0, h);
            if (u + 2 < n_mine) {
              issue_qk64(t, ks, h);
              tc_commit_w(&s_full[2 * t + h]);
              if (u + 3 == n_mine) tc_commit_w(&q_empty[t]);  // the item's last read of Q_t
            } else if (u + 2 == n_mine) {
              tc_commit_w(&pv_done[t]);   // the last sub-step's softmax has no later Q K^T to wait on
            } else {
              tc_commit_w(&o_full[t]);
            }
          }
          tc_commit_w(&k_empty[ks]);
          if (++ks == stages) { ks = 0; kph ^= 1u; }
        }
        if (!ok) break;
        continue;
      }
      if (dual) {
        // Two independent chains: K/V tile j belongs to query tile j & 1. (One item per CTA in
        // this mode, so the phases below start from zero.)
        bool ok = wait_all(&q_full[0], 0, ST_WAIT_TMA);
        for (int t = 0; t < 2 && ok; ++t) {
          if (it.n_tiles[t] == 0) continue;
          if (!wait_all(&k_full[t], 0, ST_WAIT_TMA)) { ok = false; break; }  // stages >= 2
          tc_fence_after();
          issue_qk(t, t);
          tc_commit_w(&s_full[t]);
          tc_commit_w(&k_empty[t]);
        }
        int sd = 0, sd2 = 2 % stages;                // ring slots of tiles j and j + 2
        uint32_t pd = 0, pd2 = stages == 2 ? 1 : 0;  // and the phases of their "full" barriers
        for (int j = 0; j < n_max && ok; ++j) {
          const int t = j & 1, jj = j >> 1;
          const bool more = j + 2 < n_max;
          if (!wait_all(&v_full[sd], pd, ST_WAIT_TMA)) break;
          clear_stale_v_rows(sd, it.N_ctx - (it.j0 + j) * BLOCK);
          if (more) {
            if (!wait_all(&k_full[sd2], pd2, ST_WAIT_TMA)) break;
          }
          if (!wait_all(&p_half[2 * t], jj & 1, ST_WAIT_SOFTMAX)) break;
          tc_fence_after();
          issue_pv(t, sd, jj > 0, 0);
          if (!wait_all(&p_half[2 * t + 1], jj & 1, ST_WAIT_SOFTMAX)) break;
          tc_fence_after();
          issue_pv(t, sd, jj > 0, 1);
          if (more) {
            issue_qk(t, sd2);
            tc_commit_w(&s_full[t]);
          } else {
            tc_commit_w(&o_full[t]);
          }
          tc_commit_w(&v_empty[sd]);
          if (more) tc_commit_w(&k_empty[sd2]);
          if (++sd == stages) { sd = 0; pd ^= 1; }
          if (++sd2 == stages) { sd2 = 0; pd2 ^= 1; }
        }
        break;
      }
      // Prologue: S_t = Q_t K_0^T for both tiles.
      bool ok = wait_all(&k_full[st], ph, ST_WAIT_TMA);
      for (int t = 0; t < 2 && ok; ++t) {
        if (it.n_tiles[t] == 0) continue;
        if (!wait_all(&q_full[t], q_ph[t], ST_WAIT_TMA)) { ok = false; break; }
        q_ph[t] ^= 1;
        tc_fence_after();
        issue_qk(t, st);
        tc_commit_w(&s_full[t]);
        if (it.n_tiles[t] == 1) tc_commit_w(&q_empty[t]);  // the item's last read of Q_t
      }
      if (ok) tc_commit_w(&k_empty[st]);
      for (int j = 0; j < n_max && ok; ++j) {
        const bool wrap = st + 1 == STAGES;
        const int st_next = wrap ? 0 : st + 1;
        const uint32_t ph_next = wrap ? ph ^ 1u : ph;
        if (!wait_all(&v_full[st], ph, ST_WAIT_TMA)) { ok = false; break; }
        clear_stale_v_rows(st, it.N_ctx - (it.j0 + j) * BLOCK);
        if (j + 1 < n_max) {
          if (!wait_all(&k_full[st_next], ph_next, ST_WAIT_TMA)) { ok = false; break; }
        }
        for (int t = 0; t < 2; ++t) {
          if (j >= it.n_tiles[t]) continue;
          if (!wait_all(&p_half[2 * t], p_ph[t], ST_WAIT_SOFTMAX)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, st, j > 0, 0);
          if (!wait_all(&p_half[2 * t + 1], p_ph[t], ST_WAIT_SOFTMAX)) { ok = false; break; }
          p_ph[t] ^= 1;
          tc_fence_after();
          issue_pv(t, st, j > 0, 1);
          if (j + 1 < it.n_tiles[t]) {
            issue_qk(t, st_next);
            tc_commit_w(&s_full[t]);
            if (j + 2 == it.n_tiles[t]) tc_commit_w(&q_empty[t]);  // the item's last read of Q_t
          } else {
            tc_commit_w(&o_full[t]);
          }
        }
        if (!ok) break;
        tc_commit_w(&v_empty[st]);
        if (j + 1 < n_max) tc_commit_w(&k_empty[st_next]);
        st = st_next;
        ph = ph_next;
      }
      if (!ok) break;
    }
    __syncwarp();
  } else {
    // ------------------------------------------------- softmax + epilogue warps
    reg_alloc<208>();
    const int t = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + lane_base + t * BLOCK;
    const uint32_t tmem_o = tmem_base + lane_base + 2 * BLOCK + t * D;
    const float qk_scale = args.qk_scale;
    const bool warp_idle = packed && (warp & 3) * 32 >= args.groups * args.M;
    uint32_t s_par = 0, o_par = 0;  // phases of s_full[t] and o_full[t], running on across work items
    uint32_t s_par1 = 0;            // SPLIT64: phase of the second score buffer's barrier (s_par: the first)
    uint32_t pv_idx = 0;            // SPLIT64: items of this tile so far with two or more sub-steps = phase of pv_done
    bool ok = true;

    for (int k = 0; ok; ++k) {
    const int id = item_of_round(k);
    if (id >= args.n_items || (k > 0 && *abort_flag)) break;
    const Item it = get_item(id);
    const int b = it.b, h = it.h, m0 = it.m0, j0 = it.j0, N_ctx = it.N_ctx, P_SEQ = it.P_SEQ, split = it.split;
    // Query row and head of this thread; in packed mode rows are (head, m) pairs, head-major.
    const int h_row = packed ? h + row / args.M : h;
    // (rows without a query, and tile 1 when it is unused, get the out-of-range position M)
    const int m_glob = packed ? ((row < args.groups * args.M && (dual || t == 0)) ? row % args.M : args.M)
                              : m0 + t * BLOCK + row;
    const int nt = it.n_tiles[t];
    // Keys n < lim are visible to this row.
    const int lim = (args.causal && args.d_min > -BAND_INF) ? min(N_ctx, max(0, P_SEQ + m_glob + 1 - args.d_min)) : N_ctx;
    // ... and keys n >= lo (the band's far edge).
    const int lo = (args.causal && args.d_max < BAND_INF) ? max(0, P_SEQ + m_glob + 1 - args.d_max) : 0;
    // Tiles j with (j+1)*128 <= full_upto need no masking for any row of the tile.
    const int full_upto = (args.causal && args.d_min > -BAND_INF)
                              ? min(N_ctx, max(0, P_SEQ + (packed ? 0 : m0 + t * BLOCK) + 1 - args.d_min)) : N_ctx;
    // Tiles starting at or after full_from need no masking at the far edge for any row of the tile.
    const int full_from = (args.causal && args.d_max < BAND_INF)
                              ? max(0, P_SEQ + (packed ? args.M - 1 : m0 + t * BLOCK + BLOCK - 1) + 1 - args.d_max) : 0;
    const int split_out = dual ? 2 * split + t : split;
    uint64_t ctr_row = 0;
    if constexpr (DROPOUT) {
      ctr_row = args.drop.offset +
                ((static_cast<uint64_t>(b) * args.Hq + h_row) * args.M + static_cast<uint64_t>(m_glob)) *
                    static_cast<uint64_t>(N_ctx);
    }

    float m_run = -INFINITY;
    float l_run = 0.f;

    if constexpr (SPLIT64) {
    const int n_sub = it.n_sub[t];
    for (int u = 0; u < n_sub; ++u) {
      const int bsel = u & 1;                       // score buffer of this sub-step
      const int n0 = (2 * j0 + u) * SUB;            // its first key
      uint32_t keep_bits[DROPOUT ? 2 : 1];
      if constexpr (DROPOUT) {
        const uint64_t base = ctr_row + static_cast<uint64_t>(n0);
#pragma unroll
        for (int w = 0; w < 2; ++w) keep_bits[w] = dropout_keep_word(args.drop, base + 32 * w);
        if (args.drop.keep_mask != nullptr && m_glob < args.M) {
          const int w0 = n0 >> 5;
          uint32_t* mk = args.drop.keep_mask +
                         ((static_cast<int64_t>(b) * args.Hq + h_row) * args.drop.mask_words + w0) * args.M + m_glob;
#pragma unroll
          for (int w = 0; w < 2; ++w)
            if (w0 + w < args.drop.mask_words) mk[static_cast<int64_t>(w) * args.M] = keep_bits[w];
        }
      }
      {
        const bool w = wait(&s_full[2 * t + bsel], bsel ? s_par1 : s_par);
        if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_MMA); ok = false; break; }
        if (bsel) s_par1 ^= 1; else s_par ^= 1;
      }
      tc_fence_after();
      const uint32_t tmem_sb = tmem_s + bsel * SUB;
      uint32_t s[SUB];
      tmem_ld32(tmem_sb + 0, s + 0);
      tmem_ld32(tmem_sb + 32, s + 32);
      tmem_wait_ld();

      if (n0 + SUB > full_upto || n0 < full_from) {
        // A band edge crosses these 64 keys: this row sees columns [lo_rel, hi_rel). Chunks of 32
        // columns that every row of the warp sees in full are left alone.
        const int hi_rel = lim - n0, lo_rel = lo - n0;
        const int hi_min = __reduce_min_sync(0xffffffffu, hi_rel);
        if (args.d_max >= BAND_INF) {
          // plain causal masking (no far edge): one comparison per score
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (32 * c + 32 > hi_min) {
#pragma unroll
              for (int i = 32 * c; i < 32 * c + 32; ++i)
                if (i >= hi_rel) s[i] = 0xff800000u;  // -inf
            }
          }
        } else {
          const int lo_max = __reduce_max_sync(0xffffffffu, lo_rel);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (32 * c + 32 > hi_min || 32 * c < lo_max) {
#pragma unroll
              for (int i = 32 * c; i < 32 * c + 32; ++i)
                if (i >= hi_rel || i < lo_rel) s[i] = 0xff800000u;  // -inf
            }
          }
        }
      }

      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < SUB; i += 8) {
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx0) : "f"(__uint_as_float(s[i + 0])), "f"(__uint_as_float(s[i + 1])));
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx1) : "f"(__uint_as_float(s[i + 2])), "f"(__uint_as_float(s[i + 3])));
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx2) : "f"(__uint_as_float(s[i + 4])), "f"(__uint_as_float(s[i + 5])));
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx3) : "f"(__uint_as_float(s[i + 6])), "f"(__uint_as_float(s[i + 7])));
      }
      const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));

      bool want = false;
      if (m_run == -INFINITY) {
        m_run = m_new;  // nothing accumulated yet for this row
      } else if ((m_new - m_run) * qk_scale > RESCALE_THRESHOLD) {
        want = true;
      }
      if (__any_sync(0xffffffffu, want)) {
        // The P V of the previous sub-step may still be running: wait until every P V issued for this
        // tile has completed (the next one cannot be issued before this thread has delivered its P).
        // `want` implies u >= 1, so the awaited product belongs to this item.
        // The Q K^T of sub-step u + 1 was issued right behind that P V, so its barrier (awaited again,
        // and only then consumed, at the start of the next sub-step) certifies it; behind the item's
        // second-to-last P V, where no Q K^T follows, the issuing warp commits pv_done instead.
        {
          const bool w = (u + 1 < n_sub) ? wait(&s_full[2 * t + (bsel ^ 1)], bsel ? s_par : s_par1)
                                         : wait(&pv_done[t], pv_idx & 1u);
          if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_MMA); ok = false; break; }
        }
        tc_fence_after();
        const float alpha = want ? fast_exp2((m_run - m_new) * qk_scale) : 1.0f;
        if (want) m_run = m_new;
        l_run *= alpha;
#pragma unroll
        for (int c = 0; c < D; c += 16) {
          uint32_t o[16];
          tmem_ld16(tmem_o + c, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st16(tmem_o + c, o);
        }
      }

      const float m_eff = (m_run == -INFINITY) ? 0.f : m_run;
      const float neg_ms = -m_eff * qk_scale;
      const uint64_t scale2 = f2_pack(qk_scale, qk_scale), neg_ms2 = f2_pack(neg_ms, neg_ms);
      uint64_t sum01 = 0ull, sum23 = 0ull;
#pragma unroll
      for (int i = 0; i < SUB; i += 4) {
        float p0, p1, p2, p3;
        const uint64_t x01 = f2_fma(f2_pack(__uint_as_float(s[i + 0]), __uint_as_float(s[i + 1])), scale2, neg_ms2);
        const uint64_t x23 = f2_fma(f2_pack(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), scale2, neg_ms2);
        if ((PolyMask<D>::value >> ((i >> 1) & 7)) & 1u) {
          exp2_poly_pair(x01, p0, p1);
        } else {
          float x0, x1;
          f2_unpack(x01, x0, x1);
          p0 = fast_exp2(x0);
          p1 = fast_exp2(x1);
        }
        if ((PolyMask<D>::value >> (((i >> 1) + 1) & 7)) & 1u) {
          exp2_poly_pair(x23, p2, p3);
        } else {
          float x2, x3;
          f2_unpack(x23, x2, x3);
          p2 = fast_exp2(x2);
          p3 = fast_exp2(x3);
        }
        sum01 = f2_add(sum01, f2_pack(p0, p1));
        sum23 = f2_add(sum23, f2_pack(p2, p3));
        if constexpr (DROPOUT) {
          const uint32_t kb = keep_bits[i >> 5] >> (i & 31);
          if (!(kb & 1u)) p0 = 0.f;
          if (!(kb & 2u)) p1 = 0.f;
          if (!(kb & 4u)) p2 = 0.f;
          if (!(kb & 8u)) p3 = 0.f;
        }
        s[i / 2 + 0] = pack2<BF16>(p0, p1);
        s[i / 2 + 1] = pack2<BF16>(p2, p3);
      }
      tmem_st32(tmem_sb, s);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_half[2 * t + bsel]);
      float sum0, sum1, sum2, sum3;
      f2_unpack(sum01, sum0, sum1);
      f2_unpack(sum23, sum2, sum3);
      l_run += (sum0 + sum1) + (sum2 + sum3);
    }
    if (n_sub >= 2) ++pv_idx;
    } else {
    for (int j = 0; j < nt; ++j) {
      // Dropout decisions of this row for the tile's 128 keys, generated before S is awaited so the
      // integer work overlaps the tensor core instead of extending the softmax phase.
      const int jg = j0 + (dual ? 2 * j + t : j);  // K/V tile index within the sequence
      uint32_t keep_bits[DROPOUT ? 4 : 1];
      if constexpr (DROPOUT) {
        const uint64_t base = ctr_row + static_cast<uint64_t>(jg * BLOCK);
#pragma unroll
        for (int w = 0; w < 4; ++w) keep_bits[w] = dropout_keep_word(args.drop, base + 32 * w);
        if (args.drop.keep_mask != nullptr && m_glob < args.M) {
          uint32_t* mk = args.drop.keep_mask +
                         ((static_cast<int64_t>(b) * args.Hq + h_row) * args.drop.mask_words + jg * 4) * args.M + m_glob;
#pragma unroll
          for (int w = 0; w < 4; ++w)
            if (jg * 4 + w < args.drop.mask_words) mk[static_cast<int64_t>(w) * args.M] = keep_bits[w];
        }
      }
      {
        const bool w = wait(&s_full[t], s_par);
        if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_MMA); ok = false; break; }
        s_par ^= 1;
      }
      if (warp_idle) {
        // No query row lives in this warp's 32 tile rows: keep the barrier protocol, skip the math
        // (whatever the P V product makes of these rows is never stored).
        mbar_arrive(&p_half[2 * t + 0]);
        mbar_arrive(&p_half[2 * t + 1]);
        continue;
      }
      tc_fence_after();
      uint32_t s[128];
      tmem_ld32(tmem_s + 0, s + 0);
      tmem_ld32(tmem_s + 32, s + 32);
      tmem_ld32(tmem_s + 64, s + 64);
      tmem_ld32(tmem_s + 96, s + 96);
      tmem_wait_ld();

      if ((jg + 1) * BLOCK > full_upto || jg * BLOCK < full_from) {
        // A band edge crosses the tile: this row sees tile columns [lo_rel, hi_rel). Chunks of 32
        // columns that every row of the warp sees in full are left alone (on the causal diagonal
        // that is 1.5 of a warp's 4 chunks on average; the comparisons run on the half-rate integer
        // pipe, which the softmax already loads with its conversions and maxima).
        const int hi_rel = lim - jg * BLOCK, lo_rel = lo - jg * BLOCK;
        const int hi_min = __reduce_min_sync(0xffffffffu, hi_rel);
        if (args.d_max >= BAND_INF) {
          // plain causal masking or the end of the keys (no far edge): one comparison per score
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (32 * c + 32 > hi_min) {
#pragma unroll
              for (int i = 32 * c; i < 32 * c + 32; ++i)
                if (i >= hi_rel) s[i] = 0xff800000u;  // -inf
            }
          }
        } else {
          const int lo_max = __reduce_max_sync(0xffffffffu, lo_rel);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (32 * c + 32 > hi_min || 32 * c < lo_max) {
#pragma unroll
              for (int i = 32 * c; i < 32 * c + 32; ++i)
                if (i >= hi_rel || i < lo_rel) s[i] = 0xff800000u;  // -inf
            }
          }
        }
      }

      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      // three-input max: half the instructions of a chain of two-input ones
#pragma unroll
      for (int i = 0; i < 128; i += 8) {
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx0) : "f"(__uint_as_float(s[i + 0])), "f"(__uint_as_float(s[i + 1])));
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx1) : "f"(__uint_as_float(s[i + 2])), "f"(__uint_as_float(s[i + 3])));
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx2) : "f"(__uint_as_float(s[i + 4])), "f"(__uint_as_float(s[i + 5])));
        asm("max.f32 %0, %0, %1, %2;" : "+f"(mx3) : "f"(__uint_as_float(s[i + 6])), "f"(__uint_as_float(s[i + 7])));
      }
      const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));

      // Raise the running maximum only when it moved by more than the threshold.
      bool want = false;
      if (m_run == -INFINITY) {
        m_run = m_new;  // nothing accumulated yet for this row: O row is 0 (or not yet written)
      } else if ((m_new - m_run) * qk_scale > RESCALE_THRESHOLD) {
        want = true;
      }
      if (__any_sync(0xffffffffu, want)) {
        // s_full of this iteration also certifies that P V of the previous one has completed,
        // so O is quiescent here.
        const float alpha = want ? fast_exp2((m_run - m_new) * qk_scale) : 1.0f;
        if (want) m_run = m_new;
        l_run *= alpha;
#pragma unroll
        for (int c = 0; c < D; c += 16) {
          uint32_t o[16];
          tmem_ld16(tmem_o + c, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st16(tmem_o + c, o);
        }
      }

      const float m_eff = (m_run == -INFINITY) ? 0.f : m_run;
      const float neg_ms = -m_eff * qk_scale;
      const uint64_t scale2 = f2_pack(qk_scale, qk_scale), neg_ms2 = f2_pack(neg_ms, neg_ms);
      // scale/shift, row sums and the polynomial run on packed f32x2 instructions (two scores each)
      uint64_t sum01 = 0ull, sum23 = 0ull;
      // P goes back to TMEM in two halves of 64 keys so that the P V product can start on the
      // first half while the second is still being exponentiated.
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int i = half * 64; i < half * 64 + 64; i += 4) {
          float p0, p1, p2, p3;
          const uint64_t x01 = f2_fma(f2_pack(__uint_as_float(s[i + 0]), __uint_as_float(s[i + 1])), scale2, neg_ms2);
          const uint64_t x23 = f2_fma(f2_pack(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), scale2, neg_ms2);
          if ((PolyMask<D>::value >> ((i >> 1) & 7)) & 1u) {
            exp2_poly_pair(x01, p0, p1);
          } else {
            float x0, x1;
            f2_unpack(x01, x0, x1);
            p0 = fast_exp2(x0);
            p1 = fast_exp2(x1);
          }
          if ((PolyMask<D>::value >> (((i >> 1) + 1) & 7)) & 1u) {
            exp2_poly_pair(x23, p2, p3);
          } else {
            float x2, x3;
            f2_unpack(x23, x2, x3);
            p2 = fast_exp2(x2);
            p3 = fast_exp2(x3);
          }
          sum01 = f2_add(sum01, f2_pack(p0, p1));
          sum23 = f2_add(sum23, f2_pack(p2, p3));
          if constexpr (DROPOUT) {
            const uint32_t kb = keep_bits[i >> 5] >> (i & 31);
            if (!(kb & 1u)) p0 = 0.f;
            if (!(kb & 2u)) p1 = 0.f;
            if (!(kb & 4u)) p2 = 0.f;
            if (!(kb & 8u)) p3 = 0.f;
          }
          s[i / 2 + 0] = pack2<BF16>(p0, p1);
          s[i / 2 + 1] = pack2<BF16>(p2, p3);
        }
        tmem_st32(tmem_s + half * 32, s + half * 32);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_half[2 * t + half]);
      }
      float sum0, sum1, sum2, sum3;
      f2_unpack(sum01, sum0, sum1);
      f2_unpack(sum23, sum2, sum3);
      l_run += (sum0 + sum1) + (sum2 + sum3);
    }
    }  // !SPLIT64

    // ------------------------------------------------------------- epilogue
    if (ok && nt > 0) {
      const bool w = wait(&o_full[t], o_par);
      if (!__all_sync(0xffffffffu, w)) { if (!w) fail(ST_WAIT_MMA); ok = false; }
      o_par ^= 1;
    }
    auto store_lse = [&]() {
      if (ok && m_glob < args.M) {
        const bool empty = (nt == 0) || (m_run == -INFINITY) || !(l_run > 0.f);
        const float lse = empty ? -INFINITY : m_run * args.sm_scale + logf(l_run);
        args.lse[b * args.lse_stride_b + h_row * args.lse_stride_h + split_out * args.lse_stride_split + m_glob] = lse;
      }
    };
    if (args.o_tma) {
      // 16-bit output: each thread scales its row, every warp lays its [32 x CHUNK] box out in shared
      // memory in the swizzled layout of the output tensor map (whose box is 32 rows, so that a warp
      // depends on no other warp here) and its first lane stores the box with TMA (rows past M are
      // clipped by the tensor map). The direct path below writes 32 rows x 16 bytes per warp
      // instruction, which costs several microseconds per tile.
      tc_fence_after();
      const bool empty = (nt == 0) || (m_run == -INFINITY) || !(l_run > 0.f);
      float inv = empty ? 0.f : 1.0f / l_run;
      if constexpr (DROPOUT) inv *= args.drop.inv_keep;
      const int m_warp = m0 + t * BLOCK + (warp & 3) * 32;   // first query row of this warp's box
      const bool tile_live = m_warp < args.M;                // warp-uniform
      const bool issuer = lane == 0;
      uint8_t* stage = sO + t * Cfg::CHUNK_BYTES;
      auto stage_chunk = [&](const int c) {
          uint32_t o[Cfg::CHUNK];
          if (nt > 0 && ok) {
#pragma unroll
            for (int x = 0; x < Cfg::CHUNK; x += 16) tmem_ld16(tmem_o + c * Cfg::CHUNK + x, o + x);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < Cfg::CHUNK; ++i) o[i] = 0u;
          }
          // this warp's previous store from the buffer has been read out of shared memory
          if (issuer) tma_store_wait_read();
          __syncwarp();
          const uint32_t row_addr = smem_u32(stage) + row * Cfg::ROW_BYTES;
          const uint32_t swz = (row_addr >> 7) & (Cfg::ROW_BYTES / 16 - 1);  // 16-byte unit XOR of the swizzle
#pragma unroll
          for (int u = 0; u < Cfg::ROW_BYTES / 16; ++u) {
            uint4 v;
            v.x = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * u + 0]) * inv,
                              empty ? 0.f : __uint_as_float(o[8 * u + 1]) * inv);
            v.y = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * u + 2]) * inv,
                              empty ? 0.f : __uint_as_float(o[8 * u + 3]) * inv);
            v.z = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * u + 4]) * inv,
                              empty ? 0.f : __uint_as_float(o[8 * u + 5]) * inv);
            v.w = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * u + 6]) * inv,
                              empty ? 0.f : __uint_as_float(o[8 * u + 7]) * inv);
            const uint32_t dst = row_addr + ((static_cast<uint32_t>(u) ^ swz) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                         : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (issuer && ok) {
            tma_store_4d(&tmO, stage + (warp & 3) * 32 * Cfg::ROW_BYTES, c * Cfg::CHUNK, m_warp, h, b);
            tma_store_commit();
          }
      };
      // The second chunk has to wait until the first has been read out of the staging buffer; the
      // log-normaliser fills some of that time.
      if (tile_live) stage_chunk(0);
      store_lse();
      if constexpr (Cfg::NCHUNK > 1) {
        if (tile_live) stage_chunk(1);
      }
    } else {
      store_lse();
    }
    if (!args.o_tma && ok) {
      tc_fence_after();
      const bool valid = m_glob < args.M;
      const bool empty = (nt == 0) || (m_run == -INFINITY) || !(l_run > 0.f);
      float inv = empty ? 0.f : 1.0f / l_run;
      if constexpr (DROPOUT) inv *= args.drop.inv_keep;
      const int64_t o_off = b * args.o_stride_b + h_row * args.o_stride_h + split_out * args.o_stride_split +
                            static_cast<int64_t>(m_glob) * args.o_stride_m;
#pragma unroll
      for (int c = 0; c < D; c += 16) {
        uint32_t o[16];
        __syncwarp();
        if (nt > 0) {
          tmem_ld16(tmem_o + c, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = 0u;
        }
        if (valid) {
          if (args.o_fp32) {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.o) + o_off + c);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float4 v;
              v.x = empty ? 0.f : __uint_as_float(o[4 * i + 0]) * inv;
              v.y = empty ? 0.f : __uint_as_float(o[4 * i + 1]) * inv;
              v.z = empty ? 0.f : __uint_as_float(o[4 * i + 2]) * inv;
              v.w = empty ? 0.f : __uint_as_float(o[4 * i + 3]) * inv;
              dst[i] = v;
            }
          } else {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.o) + o_off + c);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              uint4 v;
              v.x = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * i + 0]) * inv,
                                empty ? 0.f : __uint_as_float(o[8 * i + 1]) * inv);
              v.y = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * i + 2]) * inv,
                                empty ? 0.f : __uint_as_float(o[8 * i + 3]) * inv);
              v.z = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * i + 4]) * inv,
                                empty ? 0.f : __uint_as_float(o[8 * i + 5]) * inv);
              v.w = pack2<BF16>(empty ? 0.f : __uint_as_float(o[8 * i + 6]) * inv,
                                empty ? 0.f : __uint_as_float(o[8 * i + 7]) * inv);
              dst[i] = v;
            }
          }
        }
      }
      // The loads of O above have completed (tcgen05.wait::ld) before this thread's next arrival on
      // p_half, which the MMA warp awaits before the next item's first P V overwrites O.
    }
    }  // work items
    // Shared memory must outlive the reads of the last output stores.
    if (args.o_tma && lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  __syncwarp();
  if (warp == 8) {
    if (*abort_flag) {
      // Give copies that may still be in flight time to land before shared memory is released.
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) {}
    }
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200attn
