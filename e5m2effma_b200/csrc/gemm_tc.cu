// Tensor-core GEMM for sm_100a: tcgen05.mma with TMA-fed shared-memory stages and FP32
// accumulators in tensor memory.  Replaces the FP32-FMA tile kernel of the reference
// (src/gemm_e5m2effma.cuh:117-233); the epilogue keeps its documented order
// (include/e5m2effma.h:27-31).
//
// Shape of the kernel
//   * One persistent CTA per SM walks over output tiles of BI rows (index i, BI = 256 or 128) by
//     128 columns (index j).  The MMA computes the transposed tile: its M side -- the 128 lanes of
//     tensor memory -- is j (rows of op(B)^T), its N side -- TMEM columns -- is i.  A thread that
//     reads its TMEM lane therefore holds consecutive i of one column j, which are contiguous in
//     the column-major D: the epilogue converts in registers and stores 16 bytes at a time.
//   * Warp 0 (one elected lane) is the TMA producer: per k-block it brings a 128-row x 128-byte box
//     of op(B)^T and a BI-row x 128-byte box of op(A) into a ring of shared-memory stages, both in
//     the 128-byte-swizzled K-major layout the MMA reads.  Rows beyond m / n and bytes beyond k are
//     zero-filled by TMA, so tails need no special code (k is a multiple of 16 elements, a zero
//     byte is +0 in every operand format).
//   * Warp 1 (one elected lane) issues the MMAs: four K = 32-byte steps per stage, accumulating into
//     one of two TMEM buffers; tcgen05.commit hands the stage back to the producer and, after the
//     last k-block, the accumulator to the epilogue.
//   * Warps 2..9 are the epilogue: a warp owns the TMEM lane quadrant (warp index mod 4) and one
//     half of the tile's i range, reads 32 accumulators of its lane at a time with tcgen05.ld and
//     applies scale, bias, beta * C, amax and the conversion.  While they drain one buffer the MMA
//     warp already fills the other.
//   * FP8 x FP8 (any E5M2 / E4M3 pairing) runs kind::f8f6f4, BF16 x BF16 runs kind::f16; one stage
//     is 128 bytes of K either way (128 FP8 or 64 BF16 elements), so the two differ only in the
//     instruction descriptor and the element type of the tensor maps.
//   * FP8 x BF16 pairs (either order) also run kind::f16: products must stay exact, so the FP8
//     operand is widened to BF16, which is exact (at most 4 significant bits).  TMA brings its raw
//     bytes (8 KiB per k-block of 64) into the stage; the eight epilogue warps rewrite them as BF16 in
//     the swizzled layout that matches the operand's storage (K-major, or MN-major when it is stored
//     contiguous along m / n), fence towards the async proxy and signal the MMA warp, k-block by
//     k-block, and only then drain the tile's accumulator (mixed pairs have long K: the epilogue is
//     short next to the mainloop, and the TMA ring keeps filling meanwhile).  Measured alternatives
//     that were slower on this part: widening into tensor memory with the MMA reading its A operand
//     from there (each such MMA took ~280 clocks whatever its N), separate rings for raw and widened
//     data, CTA pairs (the extra cross-CTA signalling lengthens the per-stage chain).
//   * Few tiles, long K (a column shard of a weight-gradient GEMM: 64 tiles of K = 65536 on 148 SMs): the kernel
//     is launched as clusters of two CTAs that share one tile, each adding up one half of the k-blocks into its
//     own tensor memory.  When both are done, the second CTA writes its FP32 partial sums into the first one's
//     (now idle) stage ring through distributed shared memory, thread for thread, and the first adds them to its
//     own in a fixed order (deterministic) and runs the epilogue.  No scratch memory, no atomics.  The same is
//     done for the tiles of a last round that would keep at most half of the SMs busy (512 tiles on 148 SMs: 68 in
//     the fourth round): the persistent CTAs are launched as clusters of two, and after their own tiles the two CTAs
//     of a cluster share one of the remaining tiles.
//   * Otherwise no cluster features are used: every CTA loads its own operand boxes.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records a fault word, raises a
// block-wide abort flag that every role polls, and the CTA leaves through the common exit, where
// tensor memory is released.  e5b_gemm_fault() reads the word back.
#include "tc_common.cuh"
#include "gemm_tc2.cuh"
#include "gemm_tc3.cuh"
#include "gemm_tc4.cuh"

namespace e5b {
namespace tc {

// CONV: 0 both operands arrive ready for the MMA; 1 the i-side operand (op(A)) is FP8 and is
// widened to BF16 in shared memory; 2 the j-side operand (op(B)) is.
template <int BI, int CONV> struct Cfg {
  static constexpr int J_BYTES = BM * STAGE_K_BYTES;    // box of op(B)^T: 128 rows j
  static constexpr int I_BYTES = BI * STAGE_K_BYTES;    // box of op(A): BI rows i
  static constexpr int RAW_ROWS = CONV == 1 ? BI : (CONV == 2 ? BM : 0);
  static constexpr int RAW_BYTES = RAW_ROWS * (STAGE_K_BYTES / 2);   // 64 FP8 bytes per row and k-block
  static constexpr int STAGE_BYTES = J_BYTES + I_BYTES + RAW_BYTES;
  static constexpr int STAGES = CONV ? (BI == 256 ? 4 : 5) : (BI == 256 ? 4 : 6);   // mixed: 56 KiB / 40 KiB per stage
  static constexpr int NTHREADS = THREADS;
  static constexpr int TMEM_COLS = 2 * BI;
  // stages + barriers + slack for the 1 KiB alignment of the first stage
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 384;
};

// ---- the kernel ------------------------------------------------------------------------------
// map_i: tensor map of op(A) (rows i, box BI rows); map_j: tensor map of op(B)^T (rows j, box 128 rows).
// With CONV the map of the FP8 operand has 64-byte unswizzled boxes and lands in the raw area.
// FT: dtype of the FP8 operand that is widened (CONV != 0).
template <int BI, int KIND, int DT, int CONV, int FT>
__global__ void __launch_bounds__(Cfg<BI, CONV>::NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_i, const __grid_constant__ CUtensorMap map_j,
               const __grid_constant__ CUtensorMap map_ih, int m, int n, int k_bytes, uint32_t idesc, uint32_t idesc_half,
               OutDesc o, EpiMode md) {
  using C = Cfg<BI, CONV>;
  extern __shared__ uint8_t smem_raw[];
  // stage ring at the first 1 KiB boundary (the swizzle pattern repeats every 1024 bytes)
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *after_ring = smem_raw + (ring - smem_u32(smem_raw)) + C::STAGES * C::STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(after_ring);   // full[S], empty[S], acc_full[2], acc_empty[2], ready[S], xfer_go, xfer_done
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * C::STAGES + 6);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  const auto full_bar = [&](int s) { return bar0 + 8u * s; };
  const auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  const auto acc_full = [&](int b) { return bar0 + 8u * (2 * C::STAGES + b); };
  const auto acc_empty = [&](int b) { return bar0 + 8u * (2 * C::STAGES + 2 + b); };
  const auto ready_bar = [&](int s) { return bar0 + 8u * (2 * C::STAGES + 4 + s); };   // converted operand in place
  const uint32_t xfer_go = bar0 + 8u * (3 * C::STAGES + 4), xfer_done = xfer_go + 8u;  // K split over a CTA pair

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_i = (m + BI - 1) / BI, tiles_j = (n + BM - 1) / BM, tiles = tiles_i * tiles_j;
  const int kblocks_all = (k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
  // K split (md.ksplit: 1 every tile, 2 the tiles of the last, partly filled round): the two CTAs of a cluster take
  // the same tile and one half of its k-blocks each; such a tile is the last item of both CTAs
  const int ksmode = md.ksplit;
  const uint32_t crank = ksmode ? cluster_rank() : 0u;

  // Work items.  Normally one item = one tile, dealt round-robin to the CTAs.  When the last round would
  // keep at most half of the CTAs busy, its tiles are cut into two half tiles (BI / 2 rows: map_ih boxes,
  // idesc_half) so that the round takes half as long.  Every role derives the same list from this.
  const int grid_n = gridDim.x;
  const int full_items = ksmode == 1 ? 0 : (tiles / grid_n) * grid_n, rem = tiles - full_items;
  const bool split = md.split && ksmode == 0 && rem > 0 && 2 * rem <= grid_n;
  const int items = ksmode ? full_items : (split ? full_items + 2 * rem : tiles);   // dealt round-robin to single CTAs
  // this CTA's sequence: its share of `items`, then (K split) the tile full_items + cluster index shared with the peer
  const int my_main = (int)blockIdx.x < items ? (items - 1 - (int)blockIdx.x) / grid_n + 1 : 0;
  const int my_items = my_main + (ksmode && (int)(blockIdx.x >> 1) < rem ? 1 : 0);
  const auto seq_at = [&](int q, int &t, bool &shared, int &kb_first, int &kblocks) {
    shared = q >= my_main;
    t = shared ? full_items + (int)(blockIdx.x >> 1) : (int)blockIdx.x + q * grid_n;
    kb_first = shared && crank ? kblocks_all / 2 : 0;
    kblocks = shared ? (crank ? kblocks_all - kblocks_all / 2 : kblocks_all / 2) : kblocks_all;
  };
  const auto item_at = [&](int item, int &i0, int &j0, int &rows) {
    int tile = item, hf = 0;
    rows = BI;
    if (split && item >= full_items) { const int h = item - full_items; tile = full_items + (h >> 1); hf = h & 1; rows = BI / 2; }
    int ti, tj;
    tile_coords(tile, tiles_i, tiles_j, ti, tj);
    i0 = ti * BI + hf * (BI / 2);
    j0 = tj * BM;
  };

  if (threadIdx.x == 32) { prefetch_map(&map_i); prefetch_map(&map_j); prefetch_map(&map_ih); }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(ready_bar(s), EPI_WARPS / md.wgroups); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), EPI_WARPS); }
    mbar_init(xfer_go, 1);
    mbar_init(xfer_done, 32 * EPI_WARPS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {   // one warp allocates (and later frees) the accumulator columns
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (ksmode) cluster_sync_all();      // both CTAs' barriers exist before either signals the other
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int q = 0; q < my_items && ok; ++q) {
        int t, kb_first, kblocks, i0, j0, rows;
        bool shared;
        seq_at(q, t, shared, kb_first, kblocks);
        item_at(t, i0, j0, rows);
        const bool half_tile = rows != BI;
        // successive tiles of a CTA walk K in opposite directions: the next tile starts with the k-blocks that
        // were read last and are still in L2 (the sum does not care about the order of its k-blocks)
        const bool backwards = !shared && (q & 1) != 0;
        for (int kq = 0; kq < kblocks; ++kq, ++it) {
          const int kb = kb_first + (backwards ? kblocks - 1 - kq : kq);
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, (1u << 24) | (uint32_t)kb)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), C::J_BYTES + (half_tile ? C::I_BYTES / 2 : C::I_BYTES) + C::RAW_BYTES -
                                          (CONV == 1 ? C::I_BYTES : (CONV == 2 ? C::J_BYTES : 0)));
          const uint32_t sj = ring + s * C::STAGE_BYTES, si = sj + C::J_BYTES, sraw = si + C::I_BYTES;
          // coordinates are in elements of the tensor map: the innermost one counts bytes for FP8 and
          // 2-byte elements for BF16; a k-block is 128 FP8 or 64 BF16 (and then also 64 raw FP8) elements
          const int kc = kb * (KIND == 0 ? STAGE_K_BYTES : STAGE_K_BYTES / 2);
          // K-major operand: one box of all its rows.  MN-major operand: one box per 128 bytes of rows (each
          // box is a full stage of k-rows x 128 bytes), the boxes lie MN_BOX_BYTES apart.
          constexpr int EB = KIND == 0 ? 1 : 2, MN_BOX_BYTES = (STAGE_K_BYTES / EB) * 128;
          if (CONV == 2 && md.mn_m) {
            tma_load_2d(sraw, &map_j, j0, kc, full_bar(s));     // 64 k-rows x 128 raw FP8 codes along j
          } else if (md.mn_m) {
            for (int b = 0; b < BM * EB / 128; ++b) tma_load_2d(sj + b * MN_BOX_BYTES, &map_j, j0 + b * (128 / EB), kc, full_bar(s));
          } else {
            tma_load_2d(CONV == 2 ? sraw : sj, &map_j, kc, j0, full_bar(s));
          }
          if (CONV != 1 && md.mn_n) {
            for (int b = 0; b < rows * EB / 128; ++b) tma_load_2d(si + b * MN_BOX_BYTES, &map_i, i0 + b * (128 / EB), kc, full_bar(s));
          } else {
            tma_load_2d(CONV == 1 ? sraw : si, half_tile ? &map_ih : &map_i, kc, i0, full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int q = 0; q < my_items && ok; ++q, ++lt) {
        int t, kb_first, kblocks, i0, j0, rows;
        bool shared;
        seq_at(q, t, shared, kb_first, kblocks);
        item_at(t, i0, j0, rows);
        const uint32_t idesc_t = rows != BI ? idesc_half : idesc;
        const uint32_t buf = lt & 1u, use = lt >> 1;
        if (!mbar_wait(acc_empty(buf), (use & 1u) ^ 1u, abort_flag, (2u << 24) | 0xFFFFu)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BI;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag, (2u << 24) | (uint32_t)kb)) { ok = false; break; }
          if (CONV && !mbar_wait(ready_bar(s), ph, abort_flag, (4u << 24) | (uint32_t)kb)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sj = ring + s * C::STAGE_BYTES, si = sj + C::J_BYTES;
          // K-major: stepping 32 bytes along K inside the swizzled row = +2 in the 16-byte address field.
          // MN-major: one MMA spans 32 bytes of K = 32 (FP8) or 16 (BF16) k-rows of 128 bytes = +256 / +128.
          constexpr int EB = KIND == 0 ? 1 : 2;
          constexpr uint32_t MN_BOX_BYTES = (STAGE_K_BYTES / EB) * 128, MN_STEP = (MMA_K_BYTES / EB) * 128 / 16;
          const bool mnj = CONV != 1 && md.mn_m, mni = CONV != 1 && md.mn_n;
          const uint64_t dj = mnj ? mnmajor_sw128_desc(sj, MN_BOX_BYTES) : kmajor_sw128_desc(sj);
          const uint64_t di = mni ? mnmajor_sw128_desc(si, MN_BOX_BYTES) : kmajor_sw128_desc(si);
          const uint32_t stepj = mnj ? MN_STEP : 2u, stepi = mni ? MN_STEP : 2u;
#pragma unroll
          for (int ks = 0; ks < STAGE_K_BYTES / MMA_K_BYTES; ++ks)
            mma_ss<KIND>(d_tmem, dj + stepj * ks, di + stepi * ks, idesc_t, (kb | ks) != 0);
          mma_commit(empty_bar(s));
        }
        if (ok) mma_commit(acc_full(buf));
      }
    }
  } else {
    // ------------- epilogue warps: TMEM lane quadrant = warp % 4, half of the i range = (warp - 2) / 4 -------------
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const OutScalars r = out_begin(o);
    const float as_const = __fmul_rn(o.alpha, o.sa_vec ? 1.f : ld_or_one(o.sa));
    const float sb_const = o.sb_vec ? 1.f : ld_or_one(o.sb);
    float mx = 0.f;
    uint32_t lt = 0, it = 0;
    bool ok = true;
    for (int q = 0; q < my_items && ok; ++q, ++lt) {
      int t, kb_first, kblocks, i0, j0, rows;
      bool shared;
      seq_at(q, t, shared, kb_first, kblocks);
      item_at(t, i0, j0, rows);
      if (CONV != 0) {
        // Mixed pairs: these warps first widen the FP8 operand of every k-block of the tile (widen_block), then
        // drain the accumulator.  The eight warps work as WG groups that take k-blocks in turn: one pass over a
        // k-block (wait, read, convert, write, fence, arrive) is a chain of dependent latencies of several hundred
        // clocks, and with all eight warps on the same k-block that chain, not the tensor pipe, set the pace of
        // the mainloop; groups overlap WG such chains.
        const int WG = md.wgroups, GT = 32 * EPI_WARPS / WG;
        const int ct = threadIdx.x - 64, grp = ct / GT, cg = ct - grp * GT;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((int)(it % (uint32_t)WG) != grp) continue;        // warp-uniform: the group is a whole number of warps
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          ok = mbar_wait(full_bar(s), ph, abort_flag, (5u << 24) | (uint32_t)kb);
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (!ok) break;
          uint8_t *stage = smem_raw + (ring - smem_u32(smem_raw)) + s * C::STAGE_BYTES;
          const uint8_t *raw = stage + C::J_BYTES + C::I_BYTES;
          uint8_t *dst = stage + (CONV == 1 ? C::J_BYTES : 0);
          const bool mn = CONV == 2 && md.mn_m;
          if (WG == 2) { if (mn) widen_block<FT, true, 128>(raw, dst, cg); else widen_block<FT, false, 128>(raw, dst, cg); }
          else { if (mn) widen_block<FT, true, 256>(raw, dst, cg); else widen_block<FT, false, 256>(raw, dst, cg); }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
          __syncwarp();
          if (lane == 0) mbar_arrive(ready_bar(s));
        }
        if (!ok) break;
      }
      const uint32_t buf = lt & 1u, use = lt >> 1;
      ok = mbar_wait(acc_full(buf), use & 1u, abort_flag, (3u << 24) | (uint32_t)warp);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int j = j0 + quad * 32 + lane;     // index along the MMA's M side: column j, or row i when transposed
      const bool col_ok = j < n;
      const float sbj = col_ok && o.sb_vec && !md.transposed ? o.sb[j] : sb_const;
      float as_i = as_const, bias_i = 0.f;     // transposed: the per-row terms of row i = j
      if (md.transposed && col_ok) {
        if (o.sa_vec) as_i = __fmul_rn(o.alpha, o.sa[j]);
        if (o.bias) bias_i = load_elem(o.bias_dtype, o.bias, (size_t)j, 1.f);
      }
      const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BI;
      // K split: the partial sums of the second CTA travel through the first CTA's stage ring, which is idle once that
      // CTA's accumulator is complete: slot (chunk * 8 + v) * 256 + thread, 16 bytes each, written and read by the same
      // thread index of the two CTAs
      const uint32_t xslot = ring + (uint32_t)(threadIdx.x - 64) * 16u;
      if (shared && crank == 0) {
        if (threadIdx.x == 64) mbar_arrive_cluster(map_to_rank(xfer_go, 1));     // my ring is free
        ok = mbar_wait_cluster(xfer_done, 0, abort_flag, (6u << 24) | (uint32_t)warp);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
      }
      if (shared && crank == 1) {
        ok = mbar_wait_cluster(xfer_go, 0, abort_flag, (7u << 24) | (uint32_t)warp);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        const uint32_t remote = map_to_rank(xslot, 0);
        int chunk = 0;
        for (int c0 = half * (BI / 2); c0 < (half + 1) * (BI / 2); c0 += 32, ++chunk) {
          if (c0 >= rows || i0 + c0 >= m) break;   // warp-uniform
          float acc[32];
          tmem_ld32(t_lane + c0, acc);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote + (uint32_t)(chunk * 8 + v) * 4096u),
                         "f"(acc[4 * v]), "f"(acc[4 * v + 1]), "f"(acc[4 * v + 2]), "f"(acc[4 * v + 3]) : "memory");
        }
        mbar_arrive_cluster(map_to_rank(xfer_done, 0));     // every thread releases its own stores
        tc_fence_before();
        continue;                                           // the first CTA runs the epilogue
      }
      int chunk = 0;
      for (int c0 = half * (BI / 2); c0 < (half + 1) * (BI / 2); c0 += 32, ++chunk) {
        if (c0 >= rows || i0 + c0 >= m) break;   // warp-uniform
        float acc[32];
        tmem_ld32(t_lane + c0, acc);
        if (shared) {
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float4 p;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(p.x), "=f"(p.y), "=f"(p.z), "=f"(p.w)
                         : "r"(xslot + (uint32_t)(chunk * 8 + v) * 4096u) : "memory");
            acc[4 * v] = __fadd_rn(acc[4 * v], p.x);
            acc[4 * v + 1] = __fadd_rn(acc[4 * v + 1], p.y);
            acc[4 * v + 2] = __fadd_rn(acc[4 * v + 2], p.z);
            acc[4 * v + 3] = __fadd_rn(acc[4 * v + 3], p.w);
          }
        }
        if (col_ok) {
          if (md.transposed) mx = fmaxf(mx, drain32_t<DT>(o, r, acc, j, i0 + c0, m, as_i, sb_const, bias_i));
          else mx = fmaxf(mx, drain32<DT>(o, r, md, acc, i0 + c0, j, m, as_const, sbj));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(buf));
      if (!md.transposed) {   // e5b_gemm_bcast: this warp's block of the tile goes to the peers (the transposed epilogue stores to them directly)
        const int rb = i0 + half * (BI / 2), re_ = i0 + (half + 1) * (BI / 2);
        const int rend = re_ < i0 + rows ? re_ : i0 + rows;
        bcast_block<DT>(o, j0 + quad * 32, n, rb, rend < m ? rend : m);
      }
    }
    if (o.amax) {
      mx = warp_max(mx);
      if (lane == 0) amax_publish(o.amax, mx);
    }
  }

  // common exit: everybody meets (with a K split: both CTAs of the pair, so that neither leaves while the other may
  // still signal it or write into its shared memory), then the allocating warp releases tensor memory
  tc_fence_before();
  __syncthreads();
  if (ksmode) cluster_sync_all();
  if (*abort_flag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before the shared memory is reused
    const unsigned long long t0 = clock64();
    while ((unsigned long long)(clock64() - t0) < 2000000ull) { }
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// Two CTAs per tile, half of K each, when that keeps more SMs busy: at most half of the SMs would have a tile, and
// the mainloop (at least 64 k-blocks) is long next to the exchange of the partial sums (~2 us).
static bool ksplit_wanted(int tiles, int kblocks, int sms) {
  const int sw = opt(OPT_TC_KSPLIT);
  if (sw == 0 || 2 * tiles > sms || kblocks < 2) return false;
  return sw == 1 || kblocks >= 64;
}

// More tiles than SMs, and the last round would keep at most half of them busy: its tiles are shared by CTA pairs
// (half of K each) instead of being cut into half tiles, which a mixed pair does not run any faster.
static bool ksplit_tail_wanted(int tiles, int kblocks, int sms) {
  const int sw = opt(OPT_TC_KSPLIT), g = sms & ~1;
  if (sw == 0 || g < 2 || tiles <= g || kblocks < 2) return false;
  const int rem = tiles % g;
  return rem > 0 && 2 * rem <= g && (sw == 1 || kblocks >= 64);
}

template <int BI, int KIND, int DT, int CONV, int FT>
static cudaError_t launch_cfg(const CUtensorMap &mi, const CUtensorMap &mj, const CUtensorMap &mih, int m, int n,
                              int k_bytes, uint32_t idesc, uint32_t idesc_half, const OutDesc &o, const EpiMode &md, int sms,
                              cudaStream_t s) {
  using C = Cfg<BI, CONV>;
  static SmemOptIn optin;
  if (const cudaError_t e = optin.ensure(gemm_tc_kernel<BI, KIND, DT, CONV, FT>, C::SMEM_BYTES)) return e;
  const int tiles = ((m + BI - 1) / BI) * ((n + BM - 1) / BM);
  int grid = tiles < sms ? tiles : sms;
  const int cap = opt(OPT_TC_GRID);   // experiments: fewer CTAs than SMs
  if (cap > 0 && cap < grid) grid = cap;
  note_route(BI == 256 ? ROUTE_TC_256 : ROUTE_TC_128);
  const int kb_all = (k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
  const int ks = ksplit_wanted(tiles, kb_all, sms) ? 1 : (cap <= 0 && ksplit_tail_wanted(tiles, kb_all, sms) ? 2 : 0);
  if (ks) {
    // K split over CTA pairs (switch TC_KSPLIT: 0 never, 1 whenever the tiles allow it).  1: one cluster of two CTAs
    // per tile.  2: persistent CTAs as usual, launched as clusters of two, which share the tiles of the last round.
    EpiMode mk = md;
    mk.ksplit = ks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ks == 1 ? 2 * tiles : (sms & ~1));
    cfg.blockDim = dim3(C::NTHREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    note_route(ks == 1 ? (BI == 256 ? ROUTE_TC_256_KSPLIT : ROUTE_TC_128_KSPLIT) : (BI == 256 ? ROUTE_TC_256_KTAIL : ROUTE_TC_128_KTAIL));
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BI, KIND, DT, CONV, FT>, mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, mk);
  }
  gemm_tc_kernel<BI, KIND, DT, CONV, FT><<<grid, C::NTHREADS, C::SMEM_BYTES, s>>>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md);
  return cudaGetLastError();
}

template <int BI, int KIND, int CONV, int FT>
static cudaError_t launch_dt(const CUtensorMap &mi, const CUtensorMap &mj, const CUtensorMap &mih, int m, int n,
                             int k_bytes, uint32_t idesc, uint32_t idesc_half, const OutDesc &o, const EpiMode &md, int sms,
                             cudaStream_t s) {
  switch (o.d_dtype) {
    case E5MA_BF16: return launch_cfg<BI, KIND, E5MA_BF16, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    case E5MA_FP32: return launch_cfg<BI, KIND, E5MA_FP32, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    case E5MA_FP16: return launch_cfg<BI, KIND, E5MA_FP16, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    case E5MA_E5M2: return launch_cfg<BI, KIND, E5MA_E5M2, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    default: return launch_cfg<BI, KIND, E5MA_E4M3, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
  }
}

template <int BI>
static cudaError_t launch_kind(int kind, int conv, int ft, const CUtensorMap &mi, const CUtensorMap &mj,
                               const CUtensorMap &mih, int m, int n, int k_bytes, uint32_t idesc, uint32_t idesc_half,
                               const OutDesc &o, const EpiMode &md, int sms, cudaStream_t s) {
  if (kind == 0) return launch_dt<BI, 0, 0, E5MA_E5M2>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
  if (conv == 0) return launch_dt<BI, 1, 0, E5MA_E5M2>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
  return ft == E5MA_E5M2 ? launch_dt<BI, 1, 2, E5MA_E5M2>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s)
                         : launch_dt<BI, 1, 2, E5MA_E4M3>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
}

}  // namespace tc

// ---- choice between the pair kernels -----------------------------------------------------------------
// A small cost model in SM clocks, fitted to measurements on B200.  The FP8 mainloop is power-bound there: the
// 256 x 256 pair kernel, the wide-tile pair kernel (25 % fewer operand bytes per FLOP) and the one-CTA kernel
// (50 % more) all retire a 256 x 256 x 128-byte k-block per SM pair in about 712 clocks where its MMAs need 512 --
// under ncu the wide kernel shows a higher SM clock and a proportionally less busy tensor pipe, the product is
// the same.  So a k-block costs 2.78 clocks per tile row whatever the kernel, and what differs between the
// plans is how the tiles fill the rounds over the SM pairs and which epilogues are exposed: the wide kernel
// pays its epilogue after every tile, the double-buffered ones only after the last.  The 256 x 256 kernel
// carries an empirical 5 % (it measures that much slower than the model on long-K problems).
struct PairPlan { int W; double clocks; bool wide; };

static double kblock_clocks(int w) { return 2.78 * w; }
static double epilogue_clocks(int w) { return 1500.0 + 5.0 * w; }

static double pair_clocks(int m, int n, int kblocks, int W, bool wide, int sms) {
  const int tiles = ((m + W - 1) / W) * ((n + 255) / 256);
  int pairs = sms / 2;
  if (tiles < pairs) pairs = tiles;
  const int rounds = tiles / pairs, rest = tiles % pairs;
  int f = 1;
  if (rest > 0 && opt(OPT_TC_SPLIT) != 0) {
    if (wide) f = tc::wide_plan(W, tiles, pairs).slices;
    else f = 4 * rest <= pairs ? 4 : (2 * rest <= pairs ? 2 : 1);
  }
  double c = rounds * (kblocks * kblock_clocks(W) + (wide ? epilogue_clocks(W) : 0.0));
  if (rest > 0) c += kblocks * kblock_clocks(W / f) + (wide ? epilogue_clocks(W / f) : 0.0);
  if (!wide) c = c * 1.05 + epilogue_clocks(W / f);
  return c;
}
// One CTA per 128 x 256 tile, double-buffered accumulator: the same clocks per k-block and SM.
static double single_clocks(int m, int n, int kblocks, int sms) {
  const int tiles = ((m + 255) / 256) * ((n + 127) / 128);
  const int rounds = (tiles + sms - 1) / sms;
  return rounds * kblocks * kblock_clocks(256) * 1.05 + epilogue_clocks(256);
}

// W = 0: not a problem for the pair kernels.  Switch TC_WIDE: 0 = only the 256 x 256 kernel, >= 64 = that width.
// Without a switch, a measured entry of the tuned table decides before the model.
static PairPlan pair_plan(int m, int n, int k, int elem_bytes, int kblocks, int sms) {
  PairPlan best = {0, 0.0, false};
  if (m < 512 || n < 512 || sms < 2) return best;
  const int forced = opt(OPT_TC_WIDE);
  if (forced < 0) {
    const int plan = tuned_gemm_plan(elem_bytes, m, n, k);
    if (plan == -1) return best;
    if (plan == 0) return PairPlan{256, pair_clocks(m, n, kblocks, 256, false, sms), false};
    if (plan >= 64 && plan <= tc::W_MAX && plan % 32 == 0) return PairPlan{plan, pair_clocks(m, n, kblocks, plan, true, sms), true};
  }
  if (forced >= 64) {
    int W = forced > tc::W_MAX ? tc::W_MAX : forced / 32 * 32;
    return PairPlan{W, pair_clocks(m, n, kblocks, W, true, sms), true};
  }
  best = PairPlan{256, pair_clocks(m, n, kblocks, 256, false, sms), false};
  if (forced != 0) {   // full-width tiles only: no narrower width has won a measurement (the tuned table can still name one)
    const double c = pair_clocks(m, n, kblocks, tc::W_MAX, true, sms);
    if (c < best.clocks) best = PairPlan{tc::W_MAX, c, true};
  }
  if (single_clocks(m, n, kblocks, sms) < best.clocks) return PairPlan{0, 0.0, false};
  return best;
}

// Blackwell tile selection (takes the place of the reference's tuned per-architecture tables,
// src/e5m2effma_tuned.h): tiles of 256 rows x 128 columns when they fill the machine or m is large,
// else 128 x 128.  Operand pairs: FP8 x FP8 -> kind::f8f6f4; BF16 x BF16 -> kind::f16; FP8 x BF16 in
// either order -> kind::f16 with the FP8 side widened in shared memory.
cudaError_t launch_gemm_tc(int a_dtype, int b_dtype, bool a_kc, bool b_kc, const uint8_t *A, int lda,
                           const uint8_t *B, int ldb, int m, int n, int k, const OutDesc &o, int sms,
                           cudaStream_t s) {
  using namespace tc;
  if (k <= 0) return cudaErrorNotSupported;
  if (a_dtype == E5MA_FP32 || b_dtype == E5MA_FP32) return cudaErrorNotSupported;
  const bool f8 = is_fp8(a_dtype) && is_fp8(b_dtype);
  const int conv = f8 ? 0 : (is_fp8(a_dtype) ? 1 : (is_fp8(b_dtype) ? 2 : 0));
  // operands stored contiguous along m / n (transa = N, transb = T) are read as MN-major MMA operands (the
  // widened FP8 operand of a mixed pair is written in that layout too); the CTA-pair kernel takes K-contiguous ones only
  const int kind = f8 ? 0 : 1;
  const int ft = conv == 1 ? a_dtype : (conv == 2 ? b_dtype : E5MA_E5M2);
  // CTA pairs (gemm_tc2.cuh, gemm_tc3.cuh) for unmixed problems with both operands K-contiguous: the plan with the
  // lowest estimated time wins (pair_plan below); the one-CTA kernel stays for everything else.
  const bool use_pair = opt(OPT_TC_PAIR) != 0;   // experiments: 0 keeps every problem on single CTAs
  const int kblocks = (k * (f8 ? 1 : 2) + STAGE_K_BYTES - 1) / STAGE_K_BYTES;
  PairPlan plan = use_pair && a_kc && b_kc && conv == 0 ? pair_plan(m, n, k, f8 ? 1 : 2, kblocks, sms) : PairPlan{0, 0.0, false};
  // An epilogue that also copies its block to peers hides that copy only behind the mainloop of a later tile.  Wide
  // tiles that fill a single round leave all of it exposed; 256 x 256 tiles over the same problem run two rounds
  // in the same mainloop time, and the first round's copies travel during the second.
  if (o.npeers > 0 && plan.wide && opt(OPT_TC_WIDE) < 0) {
    const int wide_tiles = ((m + plan.W - 1) / plan.W) * ((n + P_TILE - 1) / P_TILE);
    const int tiles256 = ((m + P_TILE - 1) / P_TILE) * ((n + P_TILE - 1) / P_TILE);
    if (wide_tiles <= sms / 2 && tiles256 > sms / 2) plan = PairPlan{P_TILE, pair_clocks(m, n, kblocks, P_TILE, false, sms), false};
  }
  if (plan.W > 0) {
    const int fi2 = f8 ? (a_dtype == E5MA_E5M2 ? 1 : 0) : 1, fj2 = f8 ? (b_dtype == E5MA_E5M2 ? 1 : 0) : 1;
    const auto vec_ok2 = [](const void *p, int ld, int dtype) {
      return ((uintptr_t)p & 15u) == 0 && ((size_t)ld * elem_bytes(dtype)) % 16 == 0;
    };
    EpiMode pm = {};
    pm.split = opt(OPT_TC_SPLIT) != 0;
    pm.vec = vec_ok2(o.d, o.ldd, o.d_dtype);
    if (o.c && !((o.c_dtype == E5MA_FP32 || o.c_dtype == E5MA_BF16) && vec_ok2(o.c, o.ldc, o.c_dtype))) pm.vec = 0;
    if (o.bias && !((o.bias_dtype == E5MA_FP32 || o.bias_dtype == E5MA_BF16) && ((uintptr_t)o.bias & 15u) == 0)) pm.vec = 0;
    if (o.sa_vec && ((uintptr_t)o.sa & 15u)) pm.vec = 0;
    if (plan.wide) {
      const int W = plan.W;
      const int tiles = ((m + W - 1) / W) * ((n + P_TILE - 1) / P_TILE);
      int pairs = sms / 2;
      if (tiles < pairs) pairs = tiles;
      const WidePlan wp = wide_plan(W, tiles, pairs);
      CUtensorMap wi[3], wj;
      // boxes of W / 4 rows for whole tiles; W / 8 and W / 16 only when the last round is sliced (they must be
      // multiples of the 8-row swizzle group; unused maps repeat the first)
      if (!make_map(&wj, B, elem_bytes(b_dtype), k, n, ldb, 128, false) ||
          !make_map(&wi[0], A, elem_bytes(a_dtype), k, m, lda, W / 4, false) ||
          !make_map(&wi[1], A, elem_bytes(a_dtype), k, m, lda, wp.slices >= 2 ? W / 8 : W / 4, false) ||
          !make_map(&wi[2], A, elem_bytes(a_dtype), k, m, lda, wp.slices == 4 ? W / 16 : W / 4, false))
        return cudaErrorNotSupported;
      const WideDescs wd = {{instr_desc(fj2, fi2, 256, W / 2), instr_desc(fj2, fi2, 256, wp.slices >= 2 ? W / 4 : W / 2),
                             instr_desc(fj2, fi2, 256, wp.slices == 4 ? W / 8 : W / 2)}};
      return f8 ? launch_pairw<0>(wi, wj, m, n, k * 1, wp, wd, o, pm, pairs, s)
                : launch_pairw<1>(wi, wj, m, n, k * 2, wp, wd, o, pm, pairs, s);
    }
    CUtensorMap pi, pj, pi2, pi4;
    if (!make_map(&pi, A, elem_bytes(a_dtype), k, m, lda, 128, false) ||
        !make_map(&pj, B, elem_bytes(b_dtype), k, n, ldb, 128, false) ||
        !make_map(&pi2, A, elem_bytes(a_dtype), k, m, lda, 64, false) ||
        !make_map(&pi4, A, elem_bytes(a_dtype), k, m, lda, 32, false))
      return cudaErrorNotSupported;
    const uint32_t pdesc = instr_desc(fj2, fi2, 256, 256);
    const PairSplit ps = {instr_desc(fj2, fi2, 256, 128), instr_desc(fj2, fi2, 256, 64)};
    return f8 ? launch_pair<0>(pi, pj, pi2, pi4, m, n, k * 1, pdesc, ps, o, pm, sms, s)
              : launch_pair<1>(pi, pj, pi2, pi4, m, n, k * 2, pdesc, ps, o, pm, sms, s);
  }
  // Mixed FP8 x BF16 pairs with both operands K-contiguous and enough 256 x 256 tiles to keep at least half of the
  // SM pairs busy can take the CTA-pair kernel of gemm_tc4.cuh (FP8 operand on the M side, so an FP8 A runs
  // transposed) -- only on request (switch MIXED_PAIR): it measures slower than the one-CTA kernel below.
  if (conv != 0 && a_kc && b_kc && opt(OPT_MIXED_PAIR) > 0 && k >= 512) {
    const bool trp = conv == 1;
    const uint8_t *pf = trp ? A : B, *pb = trp ? B : A;
    const int ldf = trp ? lda : ldb, ldbf = trp ? ldb : lda;
    const int ef = trp ? m : n, eb = trp ? n : m;                // extents along the M side (FP8) / N side (BF16)
    const int tiles = ((ef + P_TILE - 1) / P_TILE) * ((eb + P_TILE - 1) / P_TILE);
    if (ef >= 256 && eb >= 256 && (tiles >= sms / 4 || opt(OPT_MIXED_PAIR) == 2)) {
      CUtensorMap mf, mb[3];
      if (!make_map(&mf, pf, 1, k, ef, ldf, 128, true) || !make_map(&mb[0], pb, 2, k, eb, ldbf, 128, false) ||
          !make_map(&mb[1], pb, 2, k, eb, ldbf, 64, false) || !make_map(&mb[2], pb, 2, k, eb, ldbf, 32, false))
        return cudaErrorNotSupported;
      const auto vec_okx = [](const void *p, int ld, int dtype) {
        return ((uintptr_t)p & 15u) == 0 && ((size_t)ld * elem_bytes(dtype)) % 16 == 0;
      };
      EpiMode xm = {};
      xm.transposed = trp ? 1 : 0;
      xm.split = opt(OPT_TC_SPLIT) != 0;
      xm.vec = vec_okx(o.d, o.ldd, o.d_dtype);
      if (o.c && !((o.c_dtype == E5MA_FP32 || o.c_dtype == E5MA_BF16) && vec_okx(o.c, o.ldc, o.c_dtype))) xm.vec = 0;
      if (o.bias && !((o.bias_dtype == E5MA_FP32 || o.bias_dtype == E5MA_BF16) && ((uintptr_t)o.bias & 15u) == 0)) xm.vec = 0;
      if (o.sa_vec && ((uintptr_t)o.sa & 15u)) xm.vec = 0;
      const uint32_t xdesc = instr_desc(1, 1, 256, 256);
      const PairSplit xs = {instr_desc(1, 1, 256, 128), instr_desc(1, 1, 256, 64)};
      const int fdt = trp ? a_dtype : b_dtype;
      if (trp) return fdt == E5MA_E5M2 ? launch_mixpair_dt<E5MA_E5M2, true>(mf, mb, eb, ef, k, xdesc, xs, o, xm, sms, s)
                                       : launch_mixpair_dt<E5MA_E4M3, true>(mf, mb, eb, ef, k, xdesc, xs, o, xm, sms, s);
      return fdt == E5MA_E5M2 ? launch_mixpair_dt<E5MA_E5M2, false>(mf, mb, eb, ef, k, xdesc, xs, o, xm, sms, s)
                              : launch_mixpair_dt<E5MA_E4M3, false>(mf, mb, eb, ef, k, xdesc, xs, o, xm, sms, s);
    }
  }
  // Mixed pairs widen their FP8 operand in shared memory; that costs least when the FP8 operand sits on the
  // MMA's M side (128 rows per tile instead of 256).  The M side is op(B)^T, so an FP8 A is handled by
  // running the kernel on the transposed problem (operands and m / n swapped, transposed epilogue).
  const bool tr = conv == 1;
  const uint8_t *pn = tr ? B : A, *pm = tr ? A : B;            // N-side / M-side operand storage
  const int dn = tr ? b_dtype : a_dtype, dm = tr ? a_dtype : b_dtype;
  const int ldn = tr ? ldb : lda, ldm = tr ? lda : ldb;
  const int en = tr ? n : m, em = tr ? m : n;                  // N-side / M-side extents
  const int kconv = conv ? 2 : 0;                              // after the swap the FP8 operand is always on the M side
  const int tiles256 = ((en + 255) / 256) * ((em + BM - 1) / BM);
  const int tiles128 = ((en + 127) / 128) * ((em + BM - 1) / BM);
  // 256-row tiles would idle a quarter of the SMs -- unless two CTAs can share each of them (K split), which beats smaller tiles
  const bool underfilled = tiles256 < sms && tiles128 > tiles256 && tiles256 * 4 < sms * 3 && !(en > 128 && ksplit_wanted(tiles256, kblocks, sms));
  const bool wide = en > 128 && !underfilled && (tiles256 >= sms || en % 256 == 0 || en > 1024);
  const int bi = wide ? 256 : 128;
  CUtensorMap mi, mj, mih;   // mih: the N-side operand with half-height boxes, for the half tiles of the last round
  const bool n_kc = tr ? b_kc : a_kc, m_kc = tr ? a_kc : b_kc;   // storage of the N-side / M-side operand
  if (!(n_kc ? make_map(&mi, pn, elem_bytes(dn), k, en, ldn, bi, false) : make_map_mn(&mi, pn, elem_bytes(dn), k, en, ldn)) ||
      !(m_kc ? make_map(&mj, pm, elem_bytes(dm), k, em, ldm, BM, conv != 0) : make_map_mn(&mj, pm, elem_bytes(dm), k, em, ldm, conv != 0)) ||
      !(n_kc ? make_map(&mih, pn, elem_bytes(dn), k, en, ldn, bi / 2, false) : make_map_mn(&mih, pn, elem_bytes(dn), k, en, ldn)))
    return cudaErrorNotSupported;
  // operand formats of the instruction: FP8 codes for kind::f8f6f4 (E4M3 = 0, E5M2 = 1), BF16 = 1 for kind::f16
  const int fn_ = f8 ? (dn == E5MA_E5M2 ? 1 : 0) : 1, fm_ = f8 ? (dm == E5MA_E5M2 ? 1 : 0) : 1;
  const uint32_t idesc = instr_desc(fm_, fn_, BM, bi, !m_kc, !n_kc), idesc_half = instr_desc(fm_, fn_, BM, bi / 2, !m_kc, !n_kc);
  const int k_bytes = k * (f8 ? 1 : 2);   // bytes of K per operand row as the MMA sees it
  // 16-byte vector access in the epilogue: D (and C, bias) bases and column pitches must allow it
  const auto vec_ok = [](const void *p, int ld, int dtype) {
    return ((uintptr_t)p & 15u) == 0 && ((size_t)ld * elem_bytes(dtype)) % 16 == 0;
  };
  EpiMode md = {};
  md.transposed = tr ? 1 : 0;
  md.mn_n = n_kc ? 0 : 1;
  md.mn_m = m_kc ? 0 : 1;
  md.split = wide && opt(OPT_TC_SPLIT) != 0;
  md.wgroups = opt(OPT_WIDEN_GROUPS) == 1 ? 1 : 2;   // measured on B200: 2 groups (four measured slower)
  md.vec = vec_ok(o.d, o.ldd, o.d_dtype);
  if (o.c && !((o.c_dtype == E5MA_FP32 || o.c_dtype == E5MA_BF16) && vec_ok(o.c, o.ldc, o.c_dtype))) md.vec = 0;
  if (o.bias && !((o.bias_dtype == E5MA_FP32 || o.bias_dtype == E5MA_BF16) && ((uintptr_t)o.bias & 15u) == 0)) md.vec = 0;
  if (o.sa_vec && ((uintptr_t)o.sa & 15u)) md.vec = 0;
  return wide ? launch_kind<256>(kind, kconv, ft, mi, mj, mih, en, em, k_bytes, idesc, idesc_half, o, md, sms, s)
              : launch_kind<128>(kind, kconv, ft, mi, mj, mih, en, em, k_bytes, idesc, idesc_half, o, md, sms, s);
}

}  // namespace e5b

// Reads and clears the fault word of the tensor-core GEMM on the current device.  Waits for the whole device
// first: a copy from a symbol on the legacy stream would not wait for work on non-blocking streams.
// 0: no bounded wait ever ran out.  Declared in include/e5m2effma_b200.h.
extern "C" unsigned int e5b_gemm_fault(void) {
  unsigned int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return 0xFFFFFFFFu;
  if (cudaMemcpyFromSymbol(&v, e5b::tc::g_fault, sizeof v) != cudaSuccess) return 0xFFFFFFFFu;
  cudaMemcpyToSymbol(e5b::tc::g_fault, &zero, sizeof zero);
  const unsigned int gv = e5b::gemv_fault_read_and_clear();   // the persistent GEMV's waits are bounded the same way
  const unsigned int pv = e5b::peer_fault_read_and_clear();   // and e5b_peer_barrier's
  return v ? v : (gv ? (gv | 0x80000000u) : (pv ? (pv | 0x40000000u) : 0u));
}
