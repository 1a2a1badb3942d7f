// m-grouped GEMM for device-resident weights on PAIRS of CTAs: two SMs share one tcgen05.mma.cta_group::2 instruction of
// M = 256 x N = 256. Each CTA of the pair holds 128 rows of the activation tile, HALF of the weight tile (128 of its 256
// rows) and the 128 x 256 accumulator of its own rows in its own TMEM; the tensor core of each SM reads the other SM's
// half of the weight tile from that SM's shared memory. Per output element that halves the weight bytes an SM pulls out
// of L2 -- and L2-to-SM operand traffic is what bounds the single-CTA kernels when the weights are in HBM (both the FP8
// and the BF16 256-column kernels saturate near 9 TB/s of it).
//
// No load here is a multicast: every CTA fetches its own operands with plain tiled TMA loads; the loads of the second CTA
// signal the first CTA's mbarrier (cp.async.bulk.tensor with .cta_group::2). Only the MMA thread's tcgen05.commit goes to
// the barriers of both CTAs at once.
//
// Roles per CTA as in mgrouped_kernel.cuh: warp 0 weight producer, warp 1 activation producer, warp 2 TMEM allocation,
// warps 2 and 3 (in the first CTA of the pair only) one MMA-issuing thread each, warps 4-11 two drain warpgroups of 128
// columns each.
// Work: an item is (segment, chunk of 256 * MT rows, 256-column tile), taken by pairs in turn; CTA r of the pair owns
// rows (2 * mt + r) * 128 ... of the chunk. BF16 accumulates MT = 2 row tiles per CTA in TMEM (2 x 256 columns); FP8 and
// INT8 keep one row tile's scaled accumulators in registers and use the two 256-column TMEM slots for raw per-K-block
// products, exactly as the single-CTA register-accumulating kernel does.
//
// Every mbarrier wait is bounded (wait_bar); the two cluster-wide barriers (after set-up, before tear-down) are reached
// by every thread of both CTAs on every path.
#pragma once
#include "mgrouped_kernel.cuh"

namespace agb {

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Tiled load into this CTA's shared memory whose completion is counted on an mbarrier that may live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
template <MmaKind KIND>
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == MmaKind::F16) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
  } else if constexpr (KIND == MmaKind::F8F6F4) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
  } else {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
  }
}
// Arrive on the barrier at the same offset in BOTH CTAs of the pair once every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"(both)
               : "memory");
}
// Instruction descriptor of the pair MMA: M = 256 over the two CTAs.
__host__ __device__ constexpr uint32_t make_idesc_pair(uint32_t d_fmt, uint32_t ab_fmt, uint32_t n) {
  return (d_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

constexpr int PAIR_BN = 256;          // columns of the pair's tile
constexpr int PAIR_THREADS = 384;

template <int SA, int SB, int KA>
struct PairSmem {
  static constexpr int a_box = BM * ATOM_BYTES;                   // 128 rows x 128 B of this CTA's activation rows: one K atom
  static constexpr int b_box = (PAIR_BN / 2) * ATOM_BYTES;        // this CTA's 128 of the 256 weight rows: one K atom
  static constexpr int a_stage = KA * a_box;                      // a stage holds KA K-adjacent atoms: one barrier round trip and
  static constexpr int b_stage = KA * b_box;                      // one commit per KA x 4 MMAs
  static constexpr int a_off = 0;
  static constexpr int b_off = SA * a_stage;
  static constexpr int bar_off = b_off + SB * b_stage;
  static constexpr int num_bars = 2 * SA + 2 * SB + 8;
  static constexpr int sfb_off = bar_off + num_bars * 8;          // 8 warps x 128 floats (INT8 column scales)
  static constexpr int misc_off = sfb_off + 8 * 128 * 4;
  static constexpr int work_off = misc_off + 16;                  // work list (build_work_list): 1024 segments, 512 items
  static constexpr int seg_cap = 1024, item_cap = 512;
  static constexpr int seg_first_off = work_off + seg_cap * 12;
  static constexpr int items_off = (seg_first_off + (2 * seg_cap + 2) * 4 + 15) / 16 * 16;
  static constexpr int total = items_off + item_cap * 16;
  static constexpr int dyn_bytes = total + 1024;
};

template <Kind KIND>
__host__ __device__ constexpr int pair_tiles_per_cta() { return KindTraits<KIND>::sw_scale ? 1 : 2; }

template <Kind KIND, int SA, int SB, int KA>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
mgrouped_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using T = KindTraits<KIND>;
  using L = PairSmem<SA, SB, KA>;
  static_assert(!T::sw_scale || KA == 1, "software scaling hands every 128-byte K block to the drain");
  static_assert(!T::block_scaled, "the pair kernel serves BF16, FP8 (exact scales) and INT8");
  constexpr int MT = pair_tiles_per_cta<KIND>();               // row tiles per CTA and item
  constexpr int SLOTS = TMEM_COLS / PAIR_BN;                   // 2: accumulators (BF16) or raw products (FP8 / INT8)
  constexpr uint32_t IDESC = make_idesc_pair(T::d_fmt, T::ab_fmt, PAIR_BN);
  constexpr int COLS = PAIR_BN / 2;                            // columns per drain warpgroup
  static_assert(SB % 2 == 0 && SLOTS % 2 == 0, "alternating issuers must always meet the same stages and slots");
  using AR = ARing<SA, true>;                                  // the activation ring is split between the two issuers
  constexpr uint32_t STAGE_TX_A = 2 * L::a_stage, STAGE_TX_B = 2 * L::b_stage;   // both CTAs' loads land on the first CTA's barrier

  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem + L::a_off;
  uint8_t* smem_b = smem + L::b_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint64_t* a_full = bars;               // used in the first CTA: one arrival + the bytes of both CTAs' loads
  uint64_t* a_empty = a_full + SA;       // in both CTAs: the MMA thread commits to both
  uint64_t* b_full = a_empty + SA;
  uint64_t* b_empty = b_full + SB;
  uint64_t* tm_full = b_empty + SB;      // [4] in both CTAs
  uint64_t* tm_empty = tm_full + 4;      // [4] used in the first CTA: arrivals of both CTAs' drain warps
  float* sfb_smem = reinterpret_cast<float*>(smem + L::sfb_off);
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(smem + L::misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc_off + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();          // 0 = the CTA that issues the MMAs

  if (threadIdx.x == 0) {
    for (int i = 0; i < SA; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
    for (int i = 0; i < SB; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], T::sw_scale ? 1 : 2); }   // issuers that release a stage
    for (int i = 0; i < 4; ++i) { mbar_init(&tm_full[i], 1); mbar_init(&tm_empty[i], 2 * 8); }   // 8 drain warps per CTA
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  const WorkList work = build_work_list<L::seg_cap, L::item_cap>(p, reinterpret_cast<int*>(smem + L::work_off), reinterpret_cast<int*>(smem + L::seg_first_off),
                                                                reinterpret_cast<int4*>(smem + L::items_off), blockIdx.x >> 1, gridDim.x >> 1);
  if (warp == 2) {
    tmem_alloc_pair(tmem_base_smem, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before either signals the other
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_smem;
  const WaitCtx wc{p.status, abort_flag, p.timeout_ns};
  const int kb_count = p.kb_count;                       // 128-byte K atoms
  const int ks_count = (kb_count + KA - 1) / KA;         // stages along K (atoms past the end of K arrive as zeros and are not multiplied)
  const bool flip_ok = ks_count >= SB;   // the issuers stay within SB weight stages of each other: a chunk must be at least that long

  // the same barrier in the first CTA (where both CTAs' loads and drain arrivals are counted) and in the other CTA
  auto in_first = [&](uint64_t* bar) { return map_to_cta(smem_u32(bar), 0); };

  if (warp == 0) {
    // ===================================================================== weight producer: this CTA's half of the tile
    if (lane == 0) {
      uint32_t jt = 0;
      bool ok = true;
      ItemCursor cursor(work.segs);
      for (int wi = 0; ok; ++wi) {
        Item it;
        if (!get_item(p, work, wi, cursor, it)) break;
        if (it.rows <= 0) continue;
        const int b_row = (it.expert - p.expert_lo) * p.n + it.nt * PAIR_BN + static_cast<int>(rank) * (PAIR_BN / 2);
        for (int ks = 0; ks < ks_count && ok; ++ks, ++jt) {
          const uint32_t s = jt % SB;
          ok = wait_bar(&b_empty[s], ((jt / SB) & 1) ^ 1, wc, ST_TIMEOUT_B_EMPTY);
          if (!ok) break;
          if (rank == 0) mbar_arrive_expect_tx(&b_full[s], STAGE_TX_B);
#pragma unroll
          for (int bx = 0; bx < KA; ++bx)
            tma_load_2d_pair(smem_b + s * L::b_stage + bx * L::b_box, &tmap_b, in_first(&b_full[s]), (ks * KA + bx) * ATOM_BYTES, b_row);
        }
      }
    }
  } else if (warp == 1) {
    // ===================================================================== activation producer: this CTA's 128 rows of each tile
    if (lane == 0) {
      uint32_t it_a = 0, used0 = 0, used1 = 0, chunk_no = 0;   // steps so far: all, and per issuer (ARing); chunks so far
      bool ok = true;
      ItemCursor cursor(work.segs);
      for (int wi = 0; ok; ++wi) {
        Item it;
        if (!get_item(p, work, wi, cursor, it)) break;
        if (it.rows <= 0) continue;
        const int mc = (it.rows + 2 * BM - 1) / (2 * BM);      // 256-row tiles of the pair in this chunk (<= MT)
        const uint32_t flip = flip_ok ? (chunk_no & 1u) : 0u;
        ++chunk_no;
        for (int ks = 0; ks < ks_count && ok; ++ks) {
          for (int mt = 0; mt < mc; ++mt, ++it_a) {
            const uint32_t user = (T::sw_scale ? it_a : static_cast<uint32_t>(mt) + flip) & 1u;   // as in the issuer role
            uint32_t& used = user ? used1 : used0;
            const uint32_t s = AR::stage(user, used);
            ok = wait_bar(&a_empty[s], AR::phase(used) ^ 1, wc, ST_TIMEOUT_A_EMPTY);
            if (!ok) break;
            if (rank == 0) mbar_arrive_expect_tx(&a_full[s], STAGE_TX_A);
            const int a_row = it.row0 + (2 * mt + static_cast<int>(rank)) * BM;
#pragma unroll
            for (int bx = 0; bx < KA; ++bx)
              tma_load_2d_pair(smem_a + s * L::a_stage + bx * L::a_box, &tmap_a, in_first(&a_full[s]), (ks * KA + bx) * ATOM_BYTES, a_row);
            ++used;
          }
        }
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ===================================================================== MMA issuers (first CTA of the pair only)
    // Two issuing threads, as in the single-CTA kernel: with accumulators in TMEM each row tile belongs to one of them,
    // with register accumulators the K blocks alternate (each into its own raw slot, and each weight stage has one user).
    if (lane == 0 && rank == 0) {
      const uint32_t issuer = warp - 2;
      uint32_t it_a = 0, own = 0, jt = 0, rt = 0, slot_phase = 0, chunk_no = 0;   // own: steps this issuer has taken
      bool ok = true;
      ItemCursor cursor(work.segs);
      const uint64_t a_desc0 = make_kmajor_sw128_desc(smem_u32(smem_a));
      const uint64_t b_desc0 = make_kmajor_sw128_desc(smem_u32(smem_b));
      bool a_seen = false, b_seen = false;   // the barrier of this issuer's coming step was already complete (tested ahead)
      for (int wi = 0; ok; ++wi) {
        Item it;
        if (!get_item(p, work, wi, cursor, it)) break;
        if (it.rows <= 0) continue;
        const int mc = (it.rows + 2 * BM - 1) / (2 * BM);
        const uint32_t flip = flip_ok ? (chunk_no & 1u) : 0u;   // tile ownership alternates between chunks (see the single-CTA kernel)
        ++chunk_no;
        for (int ks = 0; ks < ks_count && ok; ++ks, ++jt) {
          const uint32_t sb = jt % SB;
          const bool b_mine = !T::sw_scale || (rt & 1u) == issuer;
          if (b_mine && !b_seen) ok = wait_bar(&b_full[sb], (jt / SB) & 1, wc, ST_TIMEOUT_B_FULL);
          b_seen = false;
          if (!ok) break;
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((sb * L::b_stage) >> 4);
          for (int mt = 0; mt < mc; ++mt, ++it_a) {
            const bool mine = ((T::sw_scale ? rt : static_cast<uint32_t>(mt) + flip) & 1u) == issuer;
            if (mine) {
              const uint32_t sa = AR::stage(issuer, own);
              if (!a_seen) ok = wait_bar(&a_full[sa], AR::phase(own), wc, ST_TIMEOUT_A_FULL);
              if (!ok) break;
              uint32_t d_col;
              if constexpr (T::sw_scale) {
                const uint32_t rs = rt % SLOTS;
                ok = wait_bar(&tm_empty[rs], ((rt / SLOTS) & 1) ^ 1, wc, ST_TIMEOUT_TM_EMPTY);
                d_col = rs * PAIR_BN;
              } else {
                if (ks == 0) ok = wait_bar(&tm_empty[mt], ((slot_phase >> mt) & 1) ^ 1, wc, ST_TIMEOUT_TM_EMPTY);
                d_col = mt * PAIR_BN;
              }
              if (!ok) break;
              // a look at this issuer's next barriers; the answers are needed only after this step's MMAs are on their way
              a_seen = mbar_test_wait(&a_full[AR::stage(issuer, own + 1)], AR::phase(own + 1));
              if constexpr (!T::sw_scale) b_seen = mbar_test_wait(&b_full[(jt + 1) % SB], ((jt + 1) / SB) & 1);   // at most one tile per K atom is this issuer's
              tc_fence_after_sync();
              const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((sa * L::a_stage) >> 4);
#pragma unroll
              for (int bx = 0; bx < KA; ++bx) {
                if (ks * KA + bx >= kb_count) break;   // past the end of K
#pragma unroll
                for (int j = 0; j < ATOM_BYTES / MMA_K_BYTES; ++j) {
                  const uint32_t acc = T::sw_scale ? (j > 0) : (ks > 0 || bx > 0 || j > 0);
                  umma_pair<T::mma>(tmem_base + d_col, a_desc + static_cast<uint64_t>((bx * L::a_box + j * MMA_K_BYTES) >> 4),
                                    b_desc + static_cast<uint64_t>((bx * L::b_box + j * MMA_K_BYTES) >> 4), IDESC, acc);
                }
              }
              umma_commit_pair(&a_empty[sa]);
              ++own;
              if constexpr (T::sw_scale) {
                umma_commit_pair(&tm_full[rt % SLOTS]);
              } else {
                if (ks == ks_count - 1) umma_commit_pair(&tm_full[mt]);
              }
            }
            if constexpr (T::sw_scale) ++rt;
          }
          if (ok && b_mine) umma_commit_pair(&b_empty[sb]);
        }
        if constexpr (!T::sw_scale) slot_phase ^= (1u << mc) - 1u;
      }
    }
  } else if (warp >= 4) {
    // ===================================================================== TMEM drain: this CTA's 128 rows, two warpgroups of 128 columns
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int col_base = ((warp - 4) >> 2) * COLS;
    uint32_t rt = 0, slot_phase = 0;
    bool ok = true;
    ItemCursor cursor(work.segs);
    auto release = [&](uint64_t* bar) {     // hand a TMEM slot back to the MMA thread (its barrier lives in the first CTA)
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(in_first(bar));
    };
    for (int wi = 0; ok; ++wi) {
      Item it;
      if (!get_item(p, work, wi, cursor, it)) break;
      if (it.rows <= 0) continue;
      const int mc = (it.rows + 2 * BM - 1) / (2 * BM);
      const int n0 = it.nt * PAIR_BN;
      const long long row_end = static_cast<long long>(it.row0) + it.rows;
      if constexpr (T::sw_scale) {
        // one row tile per item (MT = 1): its scaled accumulators stay in registers over the whole K loop
        const long long grow = static_cast<long long>(it.row0) + static_cast<int>(rank) * BM + row_in_tile;
        const bool valid = grow < row_end;
        float acc[COLS];
#pragma unroll
        for (int j = 0; j < COLS; ++j) acc[j] = 0.f;
        float* sfb_buf = sfb_smem + (warp - 4) * COLS;
        const float* sfa_row = p.sfa + grow * p.sf_k;
        // FP8 only: the 128 x 128 weight block of this warpgroup's columns; with the fused activation the columns are
        // interleaved gate / up rows of the weight, which lie in two different blocks (GemmParams::epilogue)
        const bool fused = KIND == Kind::FP8 && p.epilogue != 0;
        const int blk_g = min(fused ? (n0 + col_base) >> 8 : (n0 + col_base) >> 7, p.sfb_rows - 1);
        const int blk_u = fused ? ((p.n >> 1) + ((n0 + col_base) >> 1)) >> 7 : blk_g;
        const float* sfb_blk = p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + blk_g) * p.sf_k;
        const float* sfb_blk_u = p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + blk_u) * p.sf_k;
        float sa_next = valid ? __ldg(sfa_row) : 0.f;
        float sb_next = KIND == Kind::FP8 ? __ldg(sfb_blk) : 0.f;
        float sbu_next = KIND == Kind::FP8 ? __ldg(sfb_blk_u) : 0.f;
        for (int kb = 0; kb < kb_count && ok; ++kb, ++rt) {
          const float sa = sa_next, sb_scalar = sb_next, sb_up = sbu_next;
          if (kb + 1 < kb_count) {
            sa_next = valid ? __ldg(sfa_row + kb + 1) : 0.f;
            if constexpr (KIND == Kind::FP8) {
              sb_next = __ldg(sfb_blk + kb + 1);
              sbu_next = __ldg(sfb_blk_u + kb + 1);
            }
          }
          if constexpr (KIND == Kind::INT8) {
#pragma unroll
            for (int j = 0; j < COLS / 32; ++j) {
              const int col = n0 + col_base + j * 32 + lane;
              sfb_buf[j * 32 + lane] = col < p.n ? __ldg(p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + col) * p.sf_k + kb) : 0.f;
            }
            __syncwarp();
          }
          const uint32_t rs = rt % SLOTS;
          ok = wait_bar(&tm_full[rs], (rt / SLOTS) & 1, wc, ST_TIMEOUT_TM_FULL);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t raw_addr = lane_addr + rs * PAIR_BN + col_base;
#pragma unroll
          for (int cc = 0; cc < COLS / 16; ++cc) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(raw_addr + cc * 16, r);
            tmem_wait_ld();
            if (cc == COLS / 16 - 1) release(&tm_empty[rs]);
            if constexpr (KIND == Kind::INT8) {
              if (p.raw_dump != nullptr && valid) {
                int* dst = p.raw_dump + (static_cast<long long>(kb) * p.rows_total + grow) * p.n + n0 + col_base + cc * 16;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (n0 + col_base + cc * 16 + j < p.n) dst[j] = static_cast<int>(r[j]);
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float prod, scale;
              if constexpr (KIND == Kind::INT8) {
                prod = static_cast<float>(static_cast<int>(r[j]));
                scale = sa * sfb_buf[cc * 16 + j];
              } else {
                prod = __uint_as_float(r[j]);
                scale = sa * ((cc & 1) ? sb_up : sb_scalar);   // columns 16..31 of every 32 are up rows when fused
              }
              acc[cc * 16 + j] = fmaf(prod, scale, acc[cc * 16 + j]);
            }
          }
          if constexpr (KIND == Kind::INT8) __syncwarp();
        }
        if (ok && valid) {
#pragma unroll
          for (int cc = 0; cc < COLS / 32; ++cc) {
            uint32_t v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(acc[cc * 32 + j]);
            if (fused) store_silu_mul16(p, grow, n0 + col_base + cc * 32, v);
            else store_row32(p, grow, n0 + col_base + cc * 32, v);
          }
        }
      } else {
        for (int mt = 0; mt < mc && ok; ++mt) {
          ok = wait_bar(&tm_full[mt], (slot_phase >> mt) & 1, wc, ST_TIMEOUT_TM_FULL);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const long long grow = static_cast<long long>(it.row0) + (2 * mt + static_cast<int>(rank)) * BM + row_in_tile;
          const bool valid = grow < row_end;
          uint32_t r[COLS / 32][32];
#pragma unroll
          for (int cc = 0; cc < COLS / 32; ++cc) tmem_ld_32x32b_x32(lane_addr + mt * PAIR_BN + col_base + cc * 32, r[cc]);
#pragma unroll
          for (int cc = 0; cc < COLS / 32; ++cc) tmem_wait_ld_into(r[cc]);
          release(&tm_empty[mt]);
#pragma unroll
          for (int cc = 0; cc < COLS / 32; ++cc)
            if (valid) store_row32(p, grow, n0 + col_base + cc * 32, r[cc]);
        }
        slot_phase ^= (1u << mc) - 1u;
      }
    }
  }

  // ===================================================================== common exit: both CTAs are done before TMEM goes
  if (*abort_flag) {
    // A wait of this CTA ran out. Loads of its producers and MMAs of the pair may still be in flight, and their completion
    // is counted on barriers of the first CTA, which the second cannot wait on: give them a fixed 200 us (they take a few)
    // before shared memory and TMEM are given back.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

}  // namespace agb
